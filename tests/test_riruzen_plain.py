"""The plain Riruzen implementation against hand-made values and against itself (whole, portions, token by token),
the configuration reader, and the cache plumbing the design adds (CPU)."""
import math

import pytest
import torch

import plain_riruzen as plain
import riruzen_util as rz


def test_group_norm_by_hand():
    x = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=torch.float64)
    y = plain.group_rms_norm(x, w, 2, 0.0)
    a, b = math.sqrt(12.5), math.sqrt(2.0)
    assert torch.allclose(y, torch.tensor([[3 / a, 8 / a, 0.0, 1 / b]], dtype=torch.float64))
    assert torch.allclose(plain.group_rms_norm(x, w, 1, 1e-6), plain.rms_norm(x, w, 1e-6))


def test_taps_by_hand_and_with_history():
    h = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=torch.float64)
    w = torch.tensor([[10.0, 100.0, 1000.0]], dtype=torch.float64)          # oldest tap first, the token's own last
    out = plain.causal_taps(h, w)
    assert out.flatten().tolist() == [1000.0, 2100.0, 3210.0, 4320.0]
    # a sequence cut anywhere gives the same values when the history is handed on
    for cut in (1, 2, 3):
        first = plain.causal_taps(h[:cut], w)
        hist = torch.cat([torch.zeros(2, 1, dtype=torch.float64), h[:cut]])[-2:]
        second = plain.causal_taps(h[cut:], w, hist)
        assert torch.equal(torch.cat([first, second]), out)


def test_recurrence_by_hand():
    # one head, one channel each: S_t = f S + (1 - f) v, o = S q
    w = {"q": torch.tensor([[1.0]]), "f": torch.tensor([[0.0]]), "f.b": torch.tensor([0.0]), "lower": torch.tensor([0.5]),
         "v": torch.tensor([[2.0]]), "norm": torch.tensor([1.0]), "o": torch.tensor([[1.0]])}
    w = {k: v.double() for k, v in w.items()}
    u = torch.tensor([[1.0], [1.0]], dtype=torch.float64)
    out, S = plain.hgrn2(u, w, 1, 1, 1, 0.0)
    f = 0.5 + 0.5 * 0.5                                   # sigmoid(0) = 0.5
    s1 = (1 - f) * 2.0
    s2 = f * s1 + (1 - f) * 2.0
    assert math.isclose(S.item(), s2)
    assert torch.allclose(out.flatten(), torch.tensor([1.0, 1.0], dtype=torch.float64))     # the head norm leaves the sign of S q


def test_latent_attention_sees_exactly_the_past():
    cfg = rz.CONFIGS["P"]["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(3)
    W = 24
    w = {"dq": torch.randn(cfg["q_rank"], W, generator=g), "dq.norm": torch.ones(cfg["q_rank"]), "uq": torch.randn(cfg["heads"] * cfg["dim"], cfg["q_rank"], generator=g),
         "dkv": torch.randn(cfg["kv_rank"], W, generator=g), "dkv.norm": torch.ones(cfg["kv_rank"]), "uk": torch.randn(cfg["heads"] * cfg["dim"], cfg["kv_rank"], generator=g),
         "uv": torch.randn(cfg["heads"] * cfg["vdim"], cfg["kv_rank"], generator=g), "g": torch.randn(cfg["heads"] * cfg["vdim"], W, generator=g),
         "o": torch.randn(W, cfg["heads"] * cfg["vdim"], generator=g)}
    w = {k: v.double() for k, v in w.items()}
    u = torch.randn(9, W, generator=g).double()
    args = (cfg["heads"], cfg["dim"], cfg["vdim"], cfg["scale"], 1e-6)
    whole, lat = plain.latent_attention(u, w, *args)
    changed = u.clone()
    changed[6] += 1.0                                      # a later token must not reach an earlier output
    again, _ = plain.latent_attention(changed, w, *args)
    assert torch.equal(again[:6], whole[:6]) and not torch.allclose(again[6:], whole[6:])
    # continuing from cached latents equals the whole
    head, lat5 = plain.latent_attention(u[:5], w, *args)
    tail, _ = plain.latent_attention(u[5:], w, *args, latents_before=lat5)
    assert torch.allclose(torch.cat([head, tail]), whole, atol=1e-12)
    assert torch.equal(lat[:5], lat5)


@pytest.mark.parametrize("name", list(rz.CONFIGS))
def test_whole_portions_and_single_tokens_agree(name):
    cfg = rz.CONFIGS[name]
    w = rz.make_weights(cfg, 11)
    ids = rz.tokens(cfg, 23)
    m = plain.PlainRiruzen(cfg, w)
    whole = m.forward(ids)
    m.reset()
    cut = torch.cat([m.forward(ids[:1]), m.forward(ids[1:3]), m.forward(ids[3:10]), m.forward(ids[10:11]), m.forward(ids[11:])])
    m.reset()
    single = torch.cat([m.forward([t]) for t in ids])
    assert torch.allclose(cut, whole, atol=1e-9) and torch.allclose(single, whole, atol=1e-9)


def test_configuration_reads_every_size_and_refuses_what_it_does_not_know():
    from lucciola_b200.config import ConfigError, RiruzenConfig, resolve_architecture
    d = rz.CONFIGS["P"]
    assert resolve_architecture(d).name == "Riruzen"
    cfg = RiruzenConfig.from_dict(d)
    assert (cfg.vocab, cfg.width, cfg.max_positions, cfg.logit_scale, cfg.norm_eps, cfg.norm_groups, cfg.taps) == (211, 72, 640, 0.5, 1e-6, 3, 4)
    assert [l.type for l in cfg.layers] == ["latent_attention", "latent_attention", "hgrn2", "latent_attention", "hgrn2"]
    assert cfg.layers[1].ff is None and cfg.layers[0].kv_rank == 28 and cfg.layers[2].vdim == 40
    assert RiruzenConfig.from_dict(cfg.to_dict()) == cfg
    for broken, word in ((dict(d, layers=[dict(d["layers"][0], type="conv")]), "unknown layer type"),
                         (dict(d, layers=[dict(d["layers"][0], mlp={"kind": "experts", "ff": 8})]), "unknown kind"),
                         ({k: v for k, v in d.items() if k != "logit_scale"}, "logit_scale"),
                         (dict(d, norm={"eps": 1e-6}), "groups"),
                         (dict(d, norm={"eps": 1e-6, "groups": 5}), "multiple")):
        with pytest.raises(ConfigError, match=word):
            RiruzenConfig.from_dict(broken)


def test_the_model_asks_for_the_checkpoints_tensors():
    from lucciola_b200.config import resolve_architecture
    from lucciola_b200.parts import Runtime
    for name, d in rz.CONFIGS.items():
        arch = resolve_architecture(d)
        model = arch.build(arch.config_from_dict(d), Runtime("cpu", torch.float32))
        want = {s.name: tuple(s.shape) for s in model.all_param_specs()}
        have = {k: tuple(v.shape) for k, v in rz.make_weights(d, 0).items()}
        assert want == have, name


def test_a_block_with_state_beside_its_mixers_cache():
    """Caches that ask for several things: the groups, the views and the accounting of pages."""
    from lucciola_b200.cache.device_cache import DeviceCache, bytes_per_page
    from lucciola_b200.cache.manager import plan_groups
    from lucciola_b200.parts import KVCacheView, KVPages, StateCacheView, StateSlot
    taps = StateSlot((2, 8), torch.bfloat16)
    requests = [(taps, KVPages(1, 16, 0, shared=True)), (taps, StateSlot((2, 4, 4))), KVPages(2, 8), (taps, KVPages(1, 16, 0, shared=True))]
    groups, state_keys = plan_groups(requests)
    assert [(g.num_kv_heads, g.head_dim, g.shared, g.cache_ids) for g in groups] == [(1, 16, True, ((0, 1), (3, 1))), (2, 8, False, (2,))]
    assert state_keys == [(0, 0), (1, 0), (1, 1), (3, 0)]
    assert bytes_per_page(groups, 4, torch.bfloat16) == 2 * (2 * 1 * 4 * 16) + 2 * 2 * (2 * 4 * 8)
    cache = DeviceCache(requests, groups, 4, [6, 6], 3, torch.bfloat16, torch.device("cpu"))
    a, b = cache.views[0]
    assert isinstance(a, StateCacheView) and a.state.shape == (4, 2, 8) and a.state.dtype == torch.bfloat16
    assert isinstance(b, KVCacheView) and b.k.data_ptr() == b.v.data_ptr() and b.k.shape == (6, 1, 4, 16)
    assert cache.views[1][1].state.shape == (4, 2, 4, 4) and cache.views[1][1].state.dtype == torch.float32
    assert cache.views[2].k.data_ptr() != cache.views[2].v.data_ptr()
    assert cache.views[3][1].group == 0 and cache.views[3][1].k.data_ptr() != b.k.data_ptr()
