"""Host-side logic of the Dapupel family that needs no GPU: the registry, the configuration's checks, the parameter list, the
per-sequence state's layout, the rotation rates, and the oracle's own consistency."""
import math

import pytest
import torch

import dapupel_oracle as O


def cfg_small(streams=3, taps=3):
    return O.make_config([
        O.delta_layer(4, 2, 8, 6, 3, mlp=O.moe_mlp(6, 2, 8, limit=0.7)),
        O.latent_layer(4, 8, 4, 8, 6, 12, 0.3, base=100.0, scaling=(4.0, 16, 8.0, 1.0), mlp=O.moe_mlp(3, 1, 8)),
        O.window_layer(4, 2, 8, 0.3, 5, 4.0, 2),
    ], vocab=20, width=16, streams=streams, taps=taps)


def test_registry_and_parameter_names():
    from mlx_parallm_b200.utils import _get_classes
    cfg = cfg_small()
    Model, Args = _get_classes(cfg)
    m = Model(Args.from_dict(cfg))
    assert m.model_type == "dapupel" and m.block_style == "hyper" and m.supports_ragged and m.dense
    assert sorted(m.parameter_names()) == sorted(O.random_weights(cfg).keys())
    assert m.streams == 3 and m.canon_taps == 3
    assert m.runs[0].port2 is not None and m.runs[-1].port2 is None          # the last layer has no feed-forward
    ff = m.runs[0].mlp
    assert ff.scoring == "scores" and ff.weight_on == "input" and ff.limit == 0.7 and ff.top == 2
    lat = m.mixers[1]
    assert lat.rot_dim == 4 and lat.row == 32 and lat.window == 0 and len(lat.rate_values) == 2     # 12 + 4 values, padded to 32
    win = m.mixers[2]
    assert win.window == 5 and win.softcap == 4.0 and win.taps == 2 and win.gated and win.distance_penalty


def test_state_layout():
    """Per layer: the mixer's state and the carried inputs of both input convolutions; the windowed attention caches one buffer
    for keys and values and carries its own convolution's inputs."""
    from mlx_parallm_b200.models.base import BatchedKVCache, ConvTailState, DeltaRuleState, LatentKVCache, StateGroup, TokenState
    from mlx_parallm_b200.utils import _get_classes
    cfg = cfg_small()
    Model, Args = _get_classes(cfg)
    cache = Model(Args.from_dict(cfg)).new_cache(2)
    assert len(cache) == 4 and isinstance(cache[-1], TokenState)
    kinds = (DeltaRuleState, LatentKVCache, StateGroup)
    for entry, kind in zip(cache[:3], kinds):
        assert isinstance(entry, StateGroup) and isinstance(entry.parts[0], kind)
        assert all(isinstance(p, ConvTailState) and p.channels == 16 and p.taps == 3 for p in entry.parts[1:])
    assert cache[1].parts[0].rank == 32
    kv, tail = cache[2].parts[0].parts
    assert isinstance(kv, BatchedKVCache) and kv.values_are_keys and isinstance(tail, ConvTailState) and tail.channels == (4 + 2) * 8
    kv.ensure_capacity(10, torch.float32, "cpu")
    assert kv.values is kv.keys and kv.keys.shape == (2, 2, 256, 8)
    kv._offsets = [10, 3]
    kv.ensure_capacity(300, torch.float32, "cpu")
    assert kv.values is kv.keys and kv.capacity >= 300


def test_config_checks():
    from mlx_parallm_b200.utils import _get_classes
    cfg = cfg_small()
    Model, Args = _get_classes(cfg)
    with pytest.raises(NotImplementedError):
        Args.from_dict(dict(cfg, layers=[dict(cfg["layers"][0], type="mamba2")]))
    with pytest.raises(NotImplementedError):
        Args.from_dict(dict(cfg, layers=[dict(cfg["layers"][0], mlp={"kind": "dense", "ff": 8})]))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, streams=0))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, streams=9))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, canon={"taps": 0}))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, layers=[O.window_layer(3, 2, 8, 0.3, 5, 4.0, 2)]))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, layers=[O.delta_layer(3, 2, 8, 8, 2)]))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, layers=[O.latent_layer(2, 8, 3, 8, 6, 12, 0.3)]))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, layers=[O.delta_layer(2, 2, 8, 8, 2, mlp=O.moe_mlp(3, 4, 8))]))
    bad = O.window_layer(2, 2, 8, 0.3, 5, 4.0, 2)
    bad["mixer"]["vdim"] = 12
    with pytest.raises(ValueError):
        Model(Args.from_dict(dict(cfg, layers=[bad])))


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, None), (16, 5e5, (4.0, 2048, 32.0, 1.0)), (32, 250000.0, (8.0, 4096, 32.0, 1.0)),
                                                (6, 100.0, (2.0, 64, 8.0, 1.0)), (64, 10000.0, (40.0, 4096, 32.0, 1.0)), (4, 7.0, (3.0, 8, 1.0, 1.0))])
def test_rotation_rates(dims, base, scaling):
    from mlx_parallm_b200.models.dapupel import stretched_rates
    rot = {"dims": dims, "base": base}
    sc = None
    if scaling:
        sc = rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    got, mag = stretched_rates(dims, base, sc)
    want, want_mag = O.stretched_rates(rot)
    assert len(got) == dims // 2 and all(abs(a - b) <= 1e-12 * abs(b) for a, b in zip(got, want))
    assert mag == pytest.approx(want_mag, rel=1e-15)
    plain, one = stretched_rates(dims, base)
    assert one == 1.0 and plain == [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        assert mag == pytest.approx(0.1 * math.log(sc["factor"]) + 1.0)
        for f, g in zip(plain, got):
            assert f / sc["factor"] * (1 - 1e-12) <= g <= f * (1 + 1e-12)
        assert all(a >= b for a, b in zip(got, got[1:]))                     # still ordered from fast to slow
        assert abs(got[-1] - plain[-1] / sc["factor"]) < 1e-15 or dims <= 6  # the slowest pair is fully stretched


def test_oracle_prefix_property_window_and_streams():
    """The oracle is causal (a prefix gives the prefix's logits), its windowed attention forgets what leaves the window, one copy
    of the stream with an identity-like port is a plain residual sum, and the routing weight sits on the expert's input: these
    hold for any correct statement of the design and guard the oracle itself."""
    cfg = cfg_small()
    w = O.random_weights(cfg, 1)
    t = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    full = O.forward(cfg, w, t)
    assert (O.forward(cfg, w, t[:6]) - full[:6]).abs().max() < 1e-9
    P = {k: v.double() for k, v in w.items()}
    m = dict(cfg["layers"][2]["mixer"], conv=1)
    P["l2.mix.q.conv"], P["l2.mix.k.conv"] = P["l2.mix.q.conv"][:, -1:], P["l2.mix.k.conv"][:, -1:]
    h = torch.randn(12, 16, dtype=O.F64)
    a = O.capped_window_attention(h, P, "l2.mix.", m, 1e-5)
    h2 = h.clone()
    h2[:3] = torch.randn(3, 16, dtype=O.F64)
    b = O.capped_window_attention(h2, P, "l2.mix.", m, 1e-5)
    assert (a[7:] - b[7:]).abs().max() < 1e-12 and (a[:7] - b[:7]).abs().max() > 1e-4       # window 5: position 7 sees 3..7
    one = {"hc.in": torch.ones(1, dtype=O.F64), "hc.out": torch.ones(1, dtype=O.F64), "hc.mix": torch.ones(1, 1, dtype=O.F64)}
    xs, y = torch.randn(1, 5, 8, dtype=O.F64), torch.randn(5, 8, dtype=O.F64)
    assert torch.equal(O.hyper_read(xs, one, "hc"), xs[0]) and torch.equal(O.hyper_write(xs, y, one, "hc")[0], xs[0] + y)
    mlp = cfg["layers"][0]["mlp"]
    ids, wts = O.route(h, P, "l0.mlp.", mlp["router"])
    assert ids.shape == (12, 2) and (wts > 0).all() and (wts < 1).all() and (wts[:, 0] >= wts[:, 1]).all()
    got = O.routed_ff(h, P, "l0.mlp.", mlp)
    want = sum(O.clamped_expert(wts[0, k] * h[:1], P, f"l0.mlp.e{int(ids[0, k])}.", 0.7)[0] for k in range(2))
    assert (got[0] - want).abs().max() < 1e-12
