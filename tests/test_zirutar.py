"""Zirutar through the framework against the plain implementation (plain_zirutar.py): configuration and names, cache groups, each
mechanism alone (models of one kind of layer, and the recurrence's kernels by themselves), and the engine's step function under
every way of cutting the work.  The ``gpu`` tests run the kernels; the others need no device."""
from __future__ import annotations

import json
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_zirutar
import trace_tools
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.cache import CacheManager
from tinyllama_inference_engine_b200.config import load_model_config
from tinyllama_inference_engine_b200.engine.batch import StepEntry
from tinyllama_inference_engine_b200.engine.runner import ModelRunner
from tinyllama_inference_engine_b200.errors import ConfigError
from tinyllama_inference_engine_b200.models import cache_needs, expected_tensors
from tinyllama_inference_engine_b200.models.zirutar_config import ZirutarConfig
from tinyllama_inference_engine_b200.weights import SafetensorsFile, write_random_model, write_safetensors


def _mlp(ff, limit=1.25):
    return None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}


def _attention(heads, kv_heads, dim, window, keep, mlp=None, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale if scale is not None else 2.0 * dim ** -0.5}
    if window:
        mixer["mask"] = {"size": window, "keep_first": keep}
    return {"type": "attention", "mixer": mixer, "mlp": _mlp(mlp)}


def _latent(heads, dim, rot, vdim, rank, mlp=None, base=10000.0, scale=None):
    return {"type": "latent_attention", "mlp": _mlp(mlp), "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank,
            "scale": scale if scale is not None else (dim + rot) ** -0.5, "rot": {"base": base, "dims": rot}}}


def _delta(heads, kv_heads, dim, vdim, taps, mlp=None, ranks=(8, 16)):
    return {"type": "channel_delta", "mlp": _mlp(mlp), "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps,
            "decay_rank": ranks[0], "gate_rank": ranks[1]}}


def _config(width, vocab, layers, loop=None, side=None, eps=1e-5, embed_scale=None, logit_scale=0.5):
    embed_scale = width ** 0.5 if embed_scale is None else embed_scale      # a stream well above the unit-size branches that join it, as in a trained model
    data = {"architecture": "Zirutar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "logit_scale": logit_scale, "layers": layers}
    if loop:
        data["loop"] = dict(zip(("start", "stop", "times"), loop))
    if side:
        data["token_side"] = {"dim": side}
    return data


# Sizes that agree nowhere: grouped and ungrouped heads, windows below, at and above a page (16 here), kept tokens beyond a page and none,
# rot parts of 2 to 16, ranks and widths that are multiples of 16 (the tensor-core kernels' sizes) and not, one head, convolutions of 2 to 4 taps, layers with and without a
# feed-forward, a repeated run in the middle, over the whole model, and none, with and without the second token table.
CONFIGS = {
    "all": (_config(64, 97, [_attention(4, 2, 16, 20, 3, mlp=48), _latent(3, 16, 8, 24, 32, mlp=40), _delta(4, 2, 24, 16, 3), _attention(2, 2, 32, 16, 0)],
                    loop=(1, 3, 3), side=8), 3),
    "plain_order": (_config(48, 61, [_delta(2, 1, 40, 8, 2, mlp=32, ranks=(16, 8)), _latent(1, 8, 4, 8, 16), _attention(6, 1, 16, 1, 5, mlp=24)], eps=1e-6, logit_scale=1.0), 5),
    "whole_loop": (_config(40, 53, [_attention(1, 1, 16, 24, 20, mlp=24), _delta(1, 1, 16, 8, 4), _latent(2, 16, 2, 16, 8, mlp=16, base=500.0)], loop=(0, 3, 2), side=4, embed_scale=5.0), 9),
    "attention_only": (_config(32, 50, [_attention(4, 4, 8, 7, 2), _attention(2, 1, 16, 0, 0, mlp=16), _attention(3, 1, 16, 40, 17)]), 4),
    "latent_only": (_config(32, 50, [_latent(4, 8, 16, 8, 32, mlp=16), _latent(2, 24, 4, 12, 40)]), 6),
    "delta_only": (_config(32, 50, [_delta(2, 2, 16, 16, 4), _delta(6, 2, 12, 20, 3, mlp=16), _delta(1, 1, 72, 40, 1)], side=16), 7),
    # nothing a multiple of 8: the width, the vocabulary, the feed-forwards, the heads' widths, the low ranks, the token slice
    "odd": (_config(44, 37, [_latent(3, 12, 6, 10, 20, mlp=50), _attention(2, 2, 12, 9, 1), _delta(3, 1, 10, 6, 2, mlp=26, ranks=(5, 3))], loop=(1, 2, 2), side=3), 8),
}
LENGTHS = {"all": [1, 9, 70, 150, 33, 64, 17], "plain_order": [2, 130, 65, 16, 200], "whole_loop": [3, 40, 100, 64, 7], "attention_only": [90, 5, 48, 17],
           "latent_only": [75, 1, 130, 16], "delta_only": [200, 5, 66, 2], "odd": [70, 3, 33, 18]}
TOLERANCE = {"float32": 3e-5, "bfloat16": 2.5e-2}     # 32-bit: of a row's largest difference; bfloat16: of its root mean square over the vocabulary
RMS = {"float32": False, "bfloat16": True}             # (these models amplify rounding noise: single logits of a bfloat16 row stray several times further)


def load_plain(folder, dtype=torch.float32):
    config = json.loads((folder / "config.json").read_text())
    file = SafetensorsFile(folder / "model.safetensors")
    tensors = {name: file.tensor(name).clone().to(dtype) for name in file.names()}
    file.close()
    return config, tensors


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("zirutar")
    return {key: write_random_model(base / key, config, seed) for key, (config, seed) in CONFIGS.items()}


@pytest.fixture(scope="module")
def cases(folders):
    out = {}
    for key, folder in folders.items():
        config, tensors = load_plain(folder)
        requests = trace_tools.make_requests(config["vocab"], LENGTHS[key], seed=21)
        full = {rid: plain_zirutar.forward(config, tensors, tokens) for rid, tokens in requests.items()}
        out[key] = (folder, requests, full, max(float(v.abs().max()) for v in full.values()))
    return out


def _runner(folder, dtype, max_tokens=1024, page_size=16, requests=4):
    return ModelRunner(folder, EngineConfig(dtype=dtype, page_size=page_size, max_cache_tokens=max_tokens, max_requests=requests, max_batch_tokens=1024,
                                            device="cuda:0", poison_freed_pages=True, use_cuda_graphs=False))


def _schedules(requests, seed=3, page_size=16):
    mixed, peak = trace_tools.mixed(requests, seed=seed, page_size=page_size)
    return {"whole": (trace_tools.whole(requests), 1024), "decode": (trace_tools.tail_decode(requests), 1024), "portions": (trace_tools.portions(requests), 1024),
            "mixed": (mixed, peak)}   # a pool of exactly the peak: pages are used again, and with four slots so are the state slots


# --- configuration, registry, names, cache groups -----------------------------------------------------------------------------------
def test_configuration_round_trip_registry_and_names(folders):
    architecture, config = load_model_config(folders["all"])
    assert architecture.name == "Zirutar" and isinstance(config, ZirutarConfig)
    assert ZirutarConfig.from_dict(config.to_dict()) == config
    assert config.layers[0]["mixer"]["mask"] == {"size": 20, "keep_first": 3} and config.layers[2]["mlp"] is None and config.loop == {"start": 1, "stop": 3, "times": 3}
    spec = architecture.build_spec(config)
    names = {t.name: tuple(t.shape) for t in expected_tensors(spec)}
    assert names["embed"] == (97, 64) and names["loop.step"] == (3, 64) and names["side.embed"] == (97, 32) and names["final.norm"] == (64,) and "head" not in names
    assert names["l0.mix.q"] == (64, 64) and names["l0.mix.k"] == (32, 64) and names["l0.mix.g"] == (4, 64) and names["l0.mix.o"] == (64, 64) and "l0.mix.v" not in names
    assert names["l1.mix.q"] == (72, 64) and names["l1.mix.dkv"] == (40, 64) and names["l1.mix.dkv.norm"] == (32,) and names["l1.mix.uk"] == (48, 32)
    assert names["l1.mix.uv"] == (72, 32) and names["l1.mix.sink"] == (3,) and names["l1.mix.o"] == (64, 72)
    assert names["l2.mix.q"] == (48, 64) and names["l2.mix.q.conv"] == (48, 3) and names["l2.mix.v"] == (64, 64) and names["l2.mix.b"] == (4, 64) and names["l2.mix.A_log"] == (4,)
    assert names["l2.mix.a1"] == (8, 64) and names["l2.mix.a2"] == (96, 8) and names["l2.mix.dt_bias"] == (96,) and names["l2.mix.g2"] == (64, 16) and names["l2.mix.norm"] == (16,)
    assert names["l0.mlp.gate"] == (48, 64) and names["l0.mlp.down"] == (64, 48) and "l2.mlp.up" not in names and "l2.norm2" not in names
    assert names["l3.side.gate"] == (8, 64) and names["l3.side.proj"] == (64, 8) and names["l3.side.norm"] == (64,)
    # the order of runs: layer 0, then three passes of (vector, 1, 2), then 3; every run with a cache stream of its own
    runs = [(spec.layers[e.layer].prefix, e.cache) for e in spec.order]
    assert [p for p, _ in runs] == ["l0", "loop", "l1", "l2", "loop", "l1", "l2", "loop", "l1", "l2", "l3"] and len({c for _, c in runs}) == len(runs)
    assert plain_zirutar.layer_runs(CONFIGS["all"][0]) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]


def test_low_ranks_come_from_the_tensors_shapes(folders, tmp_path):
    """A checkpoint's config.json does not name the delta rule's low ranks: they are the row counts of ``a1`` and ``g1``."""
    data = json.loads((folders["plain_order"] / "config.json").read_text())
    for key in ("decay_rank", "gate_rank"):
        data["layers"][0]["mixer"].pop(key)
    (tmp_path / "config.json").write_text(json.dumps(data))
    (tmp_path / "model.safetensors").write_bytes((folders["plain_order"] / "model.safetensors").read_bytes())
    architecture, config = load_model_config(tmp_path)
    assert config.layers[0]["mixer"]["decay_rank"] == 16 and config.layers[0]["mixer"]["gate_rank"] == 8
    with pytest.raises(ConfigError, match="low ranks"):
        architecture.build_spec(ZirutarConfig.from_dict(data))


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="lstm"), "type"),
    (lambda c: c["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "dense"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=24), "values are the keys"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c.update(loop={"start": 2, "stop": 2, "times": 2}), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_refuses_what_the_design_lacks(change, message):
    data = json.loads(json.dumps(CONFIGS["all"][0]))
    change(data)
    with pytest.raises(ConfigError, match=message):
        ZirutarConfig.from_dict(data)


def test_cache_groups_and_kept_pages():
    """Runs of equal need share a group; a window group gives back the pages its window has passed, except those of the kept first tokens."""
    architecture, config = load_model_config_from(CONFIGS["all"][0])
    needs = cache_needs(architecture.build_spec(config))
    manager = CacheManager(needs, page_size=16, num_pages=40, max_requests=2, max_positions=4096)
    groups = [(g.need.window, g.need.keep_first, g.need.page_planes(), len(g.streams)) for g in manager.page_groups]
    assert groups == [(20, 3, ((2, 16), (2, 16)), 1), (0, 0, ((1, 40),), 3), (16, 0, ((2, 32), (2, 32)), 1)]
    assert [(g.need.state_shape, len(g.streams)) for g in manager.state_groups] == [((4 * 32 * 16 + 2 * (2 * 2 * 24 + 4 * 16),), 3)]      # the matrices' key channels padded to 32
    manager.admit("a")
    manager.reserve("a", 100)
    manager.advance("a", 100)
    kept, full, plain = (manager.records["a"].tables[i] for i in range(3))
    assert [p >= 0 for p in kept] == [True, False, False, False, False, True, True]       # page 0 holds the kept tokens; positions 81.. are in pages 5, 6
    assert all(p >= 0 for p in full) and [p >= 0 for p in plain] == [False] * 5 + [True, True]
    manager.check()
    wide = CacheManager({0: type(needs[0])("pages", window=8, planes=((1, 8), (1, 8)), keep_first=20)}, page_size=16, num_pages=9, max_requests=1, max_positions=512)
    wide.admit("b")
    wide.reserve("b", 130)
    wide.advance("b", 130)
    assert [p >= 0 for p in wide.records["b"].tables[0]] == [True, True, False, False, False, False, False, True, True]   # 20 kept tokens: two pages stay


def load_model_config_from(data):
    from tinyllama_inference_engine_b200.config import architecture_for

    architecture = architecture_for(data)
    return architecture, architecture.config_class.from_dict(data)


# --- the plain implementation's own mechanisms --------------------------------------------------------------------------------------
def _random_weights(shapes, seed):
    g = torch.Generator().manual_seed(seed)
    return {name: torch.randn(shape, generator=g, dtype=torch.float64) * (shape[-1] ** -0.5 if len(shape) > 1 else 1.0) for name, shape in shapes.items()}


def test_plain_window_keeps_the_first_tokens():
    """A key just outside the window changes nothing unless it is one of the kept first tokens; the values are the keys."""
    sizes = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 1.5, "mask": {"size": 4, "keep_first": 2}}
    w = _random_weights({"a.q": (16, 12), "a.k": (8, 12), "a.g": (2, 12), "a.o": (12, 16)}, 1)
    h = torch.randn(12, 12, generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    base = plain_zirutar.windowed_attention(h, w, "a", sizes, 1e-5)
    for row, seen in ((1, True), (2, False), (7, False), (8, True), (11, True)):    # row 11 sees 0, 1 and 8..11
        moved = h.clone()
        moved[row] += 1.0
        assert (not torch.equal(plain_zirutar.windowed_attention(moved, w, "a", sizes, 1e-5)[11], base[11])) == seen, row
    assert [j for j in range(12) if plain_zirutar.visible(11, j, 4, 2)] == [0, 1, 8, 9, 10, 11]
    assert [j for j in range(5) if plain_zirutar.visible(3, j, 4, 2)] == [0, 1, 2, 3]


def test_plain_sink_takes_weight_and_rotation_is_relative():
    sizes = {"heads": 2, "dim": 4, "rot_dim": 4, "vdim": 6, "kv_rank": 8, "scale": 0.4, "rot": {"base": 100.0, "dims": 4}}
    w = _random_weights({"m.q": (16, 10), "m.dkv": (12, 10), "m.dkv.norm": (8,), "m.uk": (8, 8), "m.uv": (12, 8), "m.sink": (2,), "m.o": (10, 12)}, 3)
    h = torch.randn(9, 10, generator=torch.Generator().manual_seed(4), dtype=torch.float64)
    with_sink = plain_zirutar.latent_attention(h, w, "m", sizes, 1e-5)
    w2 = dict(w, **{"m.sink": torch.full((2,), -1e9, dtype=torch.float64)})
    without = plain_zirutar.latent_attention(h, w2, "m", sizes, 1e-5)
    assert not torch.allclose(with_sink, without, atol=1e-3)
    x = torch.randn(5, 3, 4, dtype=torch.float64)
    turned = plain_zirutar.rotate_pairs(x, torch.arange(5), 100.0, 4)
    assert torch.allclose((turned * turned).sum(-1), (x * x).sum(-1)) and torch.equal(turned[0], x[0])
    later = plain_zirutar.rotate_pairs(x, torch.arange(5) + 7, 100.0, 4)
    assert torch.allclose((turned[3, 0] * turned[1, 1]).sum(), (later[3, 0] * later[1, 1]).sum())     # a score depends on the distance only


def test_plain_delta_rule_reads_its_own_write_and_forgets_by_channel():
    sizes = {"heads": 2, "kv_heads": 1, "dim": 6, "vdim": 4, "conv": 3}
    shapes = {"d.q": (6, 10), "d.k": (6, 10), "d.v": (8, 10), "d.q.conv": (6, 3), "d.k.conv": (6, 3), "d.v.conv": (8, 3), "d.b": (2, 10), "d.A_log": (2,), "d.norm": (4,),
              "d.a1": (3, 10), "d.a2": (12, 3), "d.dt_bias": (12,), "d.g1": (3, 10), "d.g2": (8, 3), "d.o": (10, 8)}
    w = _random_weights(shapes, 5)
    h = torch.randn(14, 10, generator=torch.Generator().manual_seed(6), dtype=torch.float64)
    out = plain_zirutar.channel_delta(h, w, "d", sizes, 1e-5)
    assert not torch.allclose(out[0], torch.zeros(10, dtype=torch.float64))       # the first token reads what it has just written
    moved = h.clone()
    moved[3] += 1.0
    again = plain_zirutar.channel_delta(moved, w, "d", sizes, 1e-5)
    assert torch.equal(again[:3], out[:3]) and not torch.allclose(again[13], out[13])       # causal, and the state carries
    x = torch.arange(12, dtype=torch.float64).view(6, 2)
    taps = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    conv = plain_zirutar.short_convolution(x, taps)
    assert conv[:, 1].tolist() == x[:, 1].tolist() and conv[0, 0] == 0.0 and conv[2, 0] == 100 * 4 + 10 * 2 + 0


# --- the recurrence's kernels by themselves ---------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype,atol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("heads,kv,dim,vdim,taps,lens,cuts", [(2, 2, 16, 16, 4, [37, 1, 5], [9, 1, 2]), (6, 2, 12, 20, 3, [70], [33]), (1, 1, 72, 40, 1, [3, 20], [1, 19]),
                                                          (4, 1, 128, 24, 2, [130, 2], [64, 1]), (3, 3, 40, 8, 8, [12, 30], [5, 29])])
def test_delta_rule_kernels(dtype, atol, heads, kv, dim, vdim, taps, lens, cuts):
    """Convolution, unit norms, gates, the recurrence and the gated norm against the plain functions: every request in two steps (cut at
    ``cuts``), so that the matrices and the convolution's inputs are handed over through the state, with slots in a scrambled order."""
    from tinyllama_inference_engine_b200 import ops

    g = torch.Generator().manual_seed(heads * 10 + dim)
    channels = 2 * kv * dim + heads * vdim
    tokens = sum(lens)
    rows = torch.randn(tokens, channels + heads + 5, generator=g).to(dtype)          # five columns behind beta that are not the kernel's
    decay_in = torch.randn(tokens, heads * dim, generator=g).to(dtype)
    gate = torch.randn(tokens, heads * vdim, generator=g).to(dtype)
    conv = torch.randn(channels, taps, generator=g) * taps ** -0.5
    a_log, dt_bias, weight = torch.randn(heads, generator=g) - 1.0, torch.randn(heads * dim, generator=g), 1 + 0.1 * torch.randn(vdim, generator=g)
    # plain: every request whole
    want = torch.zeros(tokens, heads * vdim, dtype=torch.float64)
    at = 0
    for n in lens:
        x = rows[at : at + n, :channels].double()
        mixed = plain_zirutar.silu(plain_zirutar.short_convolution(x, conv.double()))
        q, k, v = mixed[:, : kv * dim].view(n, kv, dim), mixed[:, kv * dim : 2 * kv * dim].view(n, kv, dim), mixed[:, 2 * kv * dim :].view(n, heads, vdim)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(rows[at : at + n, channels : channels + heads].double())
        decay = torch.exp(-torch.exp(a_log.double()).view(1, heads, 1) * torch.nn.functional.softplus(decay_in[at : at + n].double() + dt_bias.double()).view(n, heads, dim))
        for head in range(heads):
            S = torch.zeros(dim, vdim, dtype=torch.float64)
            for t in range(n):
                S = decay[t, head].unsqueeze(1) * S
                u = beta[t, head] * (v[t, head] - S.T @ k[t, head // (heads // kv)])
                S = S + torch.outer(k[t, head // (heads // kv)], u)
                want[at + t, head * vdim : (head + 1) * vdim] = S.T @ q[t, head // (heads // kv)]
        at += n
    want = (plain_zirutar.unit_rms(want.view(tokens, heads, vdim), 1e-5) * weight.double() * torch.sigmoid(gate.double()).view(tokens, heads, vdim)).view(tokens, -1)
    # the kernels: two steps
    words, conv_offset = ops.delta_state_words(heads, dim, vdim, channels, taps)
    state = torch.full((5, words), 7.0, device="cuda")
    slots = [3, 0, 4][: len(lens)]
    state[slots] = 0.0
    got = torch.zeros(tokens, heads * vdim, dtype=dtype, device="cuda")
    starts = np.concatenate([[0], np.cumsum(lens)])
    for part in range(2):
        pieces = [(starts[i] + (0 if part == 0 else cuts[i]), cuts[i] if part == 0 else lens[i] - cuts[i]) for i in range(len(lens))]
        pieces = [(i, a, n) for i, (a, n) in enumerate(pieces) if n > 0]
        index = torch.cat([torch.arange(a, a + n) for _, a, n in pieces])
        count = [n for _, _, n in pieces]
        ctx = SimpleNamespace(num_seqs=len(pieces), token_seq=torch.tensor([j for j, n in enumerate(count) for _ in range(n)], dtype=torch.int32).cuda(),
                              seq_starts=torch.tensor(np.concatenate([[0], np.cumsum(count)]), dtype=torch.int32).cuda(),
                              state_slots=torch.tensor([slots[i] for i, _, _ in pieces], dtype=torch.int32).cuda())
        step_rows, n_rows = rows[index].cuda().contiguous(), len(index)
        prep = torch.zeros(n_rows, channels + heads + heads * dim, device="cuda")
        read = torch.zeros(n_rows, heads * vdim, device="cuda")
        out = torch.zeros(n_rows, heads * vdim, dtype=dtype, device="cuda")
        ops.delta_prepare(step_rows, channels, decay_in[index].cuda().contiguous(), conv.cuda(), a_log.cuda(), dt_bias.cuda(), state, conv_offset, ctx, prep, heads, kv, dim, vdim,
                          1e-6, dim ** -0.5)
        ops.delta_rule(prep, state, ctx, read, heads, kv, dim, vdim)
        ops.delta_gate_norm(read, gate[index].cuda().contiguous(), weight.cuda(), out, 1e-5, heads, vdim)
        got[index.cuda()] = out
    assert float((got.cpu().double() - want).abs().max()) <= atol * max(1.0, float(want.abs().max()))
    untouched = [s for s in range(5) if s not in slots]
    assert bool((state[untouched] == 7.0).all())


# --- the engine on the GPU under every way of cutting the work ---------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", list(CONFIGS))
def test_engine_matches_plain_under_every_schedule(cases, key, dtype):
    """Whole prompts, a tail decoded token by token, portions down to two tokens, and four live requests mixed in a pool that makes
    pages and state slots come round again (freed pages are poisoned with NaN)."""
    folder, requests, full, scale = cases[key]
    for name, (steps, pool) in _schedules(requests).items():
        runner = _runner(folder, dtype, max_tokens=pool)
        trace_tools.run_and_compare(runner, steps, full, atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype])
        runner.cache.check()
        assert not runner.cache.records, name
        if name == "mixed":
            assert all(g.pool.reuses > 0 for g in runner.cache.page_groups)


@pytest.mark.gpu
def test_layer_outputs_match_the_plain_trace(cases):
    folder, requests, full, scale = cases["all"]
    config, tensors = load_plain(folder)
    tokens = requests["r4"]
    want = []
    plain_zirutar.forward(config, tensors, tokens, want)
    trace = {}
    _runner(folder, "float32").step([StepEntry("a", tokens, [0])], trace=trace)
    assert len(trace) == len(want) == 8          # the vectors that start a pass are no layers of their own
    for index, layer in enumerate(want):
        assert float((trace[f"layer{index}.output"].cpu() - layer).abs().max()) <= 3e-5 * float(layer.abs().max()), index


def _sharpened(folder, name, edit, config_edit=None):
    """A copy of a model folder with some tensors (and constants) changed, so that one mechanism decides the logits."""
    target = folder.parent / f"{folder.name}_{name}"
    target.mkdir(exist_ok=True)
    config = json.loads((folder / "config.json").read_text())
    if config_edit:
        config_edit(config)
    (target / "config.json").write_text(json.dumps(config))
    _, tensors = load_plain(folder, torch.bfloat16)
    edit(tensors)
    write_safetensors(target / "model.safetensors", tensors)
    return target


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_edges_and_kept_tokens_decide(folders, dtype):
    """A large score scale makes single keys dominate a row: one key too many or too few at a window's edge, or a kept first token
    that is dropped, then moves the logits far beyond the tolerance, in prompts, in portions and in decoded tokens."""
    def sharper(config):
        for layer in config["layers"]:
            layer["mixer"]["scale"] = 2.5

    folder = _sharpened(folders["attention_only"], "sharp", lambda tensors: None, sharper)
    config, tensors = load_plain(folder)
    requests = trace_tools.make_requests(config["vocab"], [130, 48, 65, 33], seed=13)
    full = {rid: plain_zirutar.forward(config, tensors, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    for change in (lambda c: c["layers"][2]["mixer"]["mask"].update(size=39), lambda c: c["layers"][2]["mixer"]["mask"].update(size=41),
                   lambda c: c["layers"][2]["mixer"]["mask"].update(keep_first=16), lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=3)):
        other = json.loads(json.dumps(config))
        change(other)
        assert float((plain_zirutar.forward(other, tensors, requests["r0"]) - full["r0"]).abs().max()) > 50 * TOLERANCE["float32"] * scale
    for steps in (trace_tools.tail_decode(requests, tail=60), trace_tools.portions(requests), trace_tools.mixed(requests, seed=6)[0]):
        trace_tools.run_and_compare(_runner(folder, dtype), steps, full, atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sinks_and_far_keys_decide(folders, dtype):
    """Large sinks take most of a row's weight, and a large score scale lets keys hundreds of tokens back win: leaving the sink out, or
    losing a far key at a page's border, shows in the logits."""
    def edit(tensors):
        for name in tensors:
            if name.endswith(".sink"):
                tensors[name] = torch.full_like(tensors[name], 3.0)

    def sharper(config):
        for layer in config["layers"]:
            layer["mixer"]["scale"] = 2.0

    folder = _sharpened(folders["latent_only"], "sinks", edit, sharper)
    config, tensors = load_plain(folder)
    requests = trace_tools.make_requests(config["vocab"], [400, 70], seed=17)
    full = {rid: plain_zirutar.forward(config, tensors, tokens) for rid, tokens in requests.items()}
    scale = max(float(v.abs().max()) for v in full.values())
    no_sinks = {name: (torch.full_like(t, -1e9) if name.endswith(".sink") else t) for name, t in tensors.items()}
    assert float((plain_zirutar.forward(config, no_sinks, requests["r1"]) - full["r1"]).abs().max()) > 50 * TOLERANCE["float32"] * scale
    early = [(t + 1) % config["vocab"] if 10 <= i < 110 else t for i, t in enumerate(requests["r0"])]       # across page borders, 290 tokens and more back
    assert float((plain_zirutar.forward(config, tensors, early)[-1] - full["r0"][-1]).abs().max()) > 50 * TOLERANCE["float32"] * scale      # keys 300 back show
    for steps in (trace_tools.tail_decode(requests, tail=40), trace_tools.portions(requests), trace_tools.mixed(requests, seed=4, max_portion=90)[0]):
        trace_tools.run_and_compare(_runner(folder, dtype, max_tokens=2048), steps, full, atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tokens_hundreds_back_decide_through_the_state(folders, dtype):
    """Decays close to one keep what the matrices took in for hundreds of steps: the last logits of a 500-token request then depend on
    its first hundred tokens, through every portion's hand-over of the state and through 150 tokens decoded one by one."""
    def slow(tensors):
        for name in tensors:
            if name.endswith(".A_log"):
                tensors[name] = torch.full_like(tensors[name], -7.0)
            if name.endswith(".dt_bias"):
                tensors[name] = torch.full_like(tensors[name], -3.0)

    folder = _sharpened(folders["delta_only"], "slow", slow)
    config, tensors = load_plain(folder)
    requests = trace_tools.make_requests(config["vocab"], [500, 320], seed=8)
    full = {rid: plain_zirutar.forward(config, tensors, tokens) for rid, tokens in requests.items()}
    other = [(t + 1) % config["vocab"] if i < 100 else t for i, t in enumerate(requests["r0"])]
    scale = max(float(v.abs().max()) for v in full.values())
    assert float((plain_zirutar.forward(config, tensors, other)[-1] - full["r0"][-1]).abs().max()) > 50 * TOLERANCE["float32"] * scale
    for steps in (trace_tools.tail_decode(requests, tail=150), trace_tools.portions(requests), trace_tools.mixed(requests, seed=4, max_portion=90)[0]):
        trace_tools.run_and_compare(_runner(folder, dtype, max_tokens=2048, page_size=64), steps, full, atol=TOLERANCE[dtype] * scale, over_vocabulary=RMS[dtype])


@pytest.mark.gpu
def test_rows_do_not_depend_on_the_batch(cases):
    """32-bit rows agree to rounding however the step is cut and whatever else is in the batch."""
    folder, requests, full, scale = cases["all"]
    alone, together = _runner(folder, "float32"), _runner(folder, "float32")
    tokens = requests["r3"]
    whole = alone.step([StepEntry("x", tokens, [len(tokens) - 1])]).cpu()
    together.step([StepEntry("y", requests["r2"][:40], []), StepEntry("x", tokens[:77], [])])
    cut = together.step([StepEntry("x", tokens[77:], [len(tokens) - 78]), StepEntry("y", requests["r2"][40:41], [0])]).cpu()
    assert float((cut[0] - whole[0]).abs().max()) <= 1e-5 * scale


# --- generation through the engine's own entry point -------------------------------------------------------------------------------------
def _plain_greedy(config, tensors, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(plain_zirutar.forward(config, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(folders, graphs):
    """Prompts of unequal length through ``Engine.generate``: scheduler, portions under a small token budget, decode sessions
    (captured as graphs or not), state slots, windowed pages with kept first tokens.  32-bit, so that the plain choice is the engine's."""
    from tinyllama_inference_engine_b200 import Engine, SamplingParams

    folder = folders["all"]
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
    prompts = [[int(t) for t in rng.integers(0, 61, size=n)] for n in (90, 12, 40)]
    first = generate(folders["plain_order"], prompts, max_tokens=24, dtype="bfloat16", page_size=16, max_cache_tokens=1024, max_requests=4, max_batch_tokens=64)
    second = generate(folders["plain_order"], prompts, max_tokens=24, dtype="bfloat16", page_size=16, max_cache_tokens=1024, max_requests=4, max_batch_tokens=64)
    assert first == second and all(len(tokens) == 24 for tokens in first)


@pytest.mark.gpu
def test_command_line_and_feed_forward_of_few_rows(folders, capsys):
    """The framework's command line generates with a Zirutar folder and prints its logits; a decode step's feed-forward (the clamped gate in
    the product's epilogue, up to 16 rows) gives what a prompt portion's does (a kernel of its own behind the product)."""
    from tinyllama_inference_engine_b200 import ops
    from tinyllama_inference_engine_b200.cli import main

    folder = folders["all"]
    config, tensors = load_plain(folder)
    prompt = [int(t) for t in np.random.default_rng(12).integers(0, config["vocab"], size=11)]
    text = ",".join(map(str, prompt))
    assert main(["generate", str(folder), text, "6", "--dtype", "float32", "--page-size", "16"]) == 0
    result = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert result["generated_tokens"] == _plain_greedy(config, tensors, prompt, 6) and result["prompt_tokens"] == 11
    assert main(["logits", str(folder), text, "--dtype", "float32"]) == 0
    logits = torch.tensor(json.loads(capsys.readouterr().out)["logits"])
    assert torch.allclose(logits, plain_zirutar.forward(config, tensors, prompt)[-1], atol=3e-5 * float(logits.abs().max()))
    g = torch.Generator().manual_seed(5)
    weight = (torch.randn(2 * 72, 64, generator=g) * 0.3).bfloat16().cuda()
    for rows in (1, 7, 16):
        x = torch.randn(rows, 64, generator=g).bfloat16().cuda()
        gate_up = torch.zeros(rows, 144, dtype=torch.bfloat16, device="cuda")
        want, got = torch.zeros(rows, 72, dtype=torch.bfloat16, device="cuda"), torch.zeros(rows, 72, dtype=torch.bfloat16, device="cuda")
        ops.linear(x, weight, gate_up)
        ops.clamped_gate_mul(gate_up, want, 0.8, 1.702, 1.0)
        before = ops.launch_count
        ops.linear_gated(x, weight, got, clamp=(0.8, 1.702, 1.0))
        assert ops.launch_count - before == 1
        assert torch.allclose(got.float(), want.float(), atol=1e-2, rtol=1e-2)
        reference = x.float().cpu() @ weight.float().cpu().T
        plain = torch.clamp(reference[:, :72], max=0.8)
        plain = plain * torch.sigmoid(1.702 * plain) * (torch.clamp(reference[:, 72:], -0.8, 0.8) + 1.0)
        assert torch.allclose(got.float().cpu(), plain, atol=3e-2, rtol=3e-2)
