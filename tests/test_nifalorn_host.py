"""Host-side logic of the Nifalorn family that needs no GPU: the registry, the configuration's checks, the order of layer runs
of a looped span, the parameter list, the rotation rates, and the oracle's own consistency."""
import math

import pytest
import torch

import nifalorn_oracle as O


def cfg_small(loop=None):
    return O.make_config([
        O.ssm_layer(2, 8, 6, 1, 2, conv=3, mlp=O.dense_mlp(16)),
        O.attention_layer(4, 2, 8, 8, 0.3, 0.4, 5, 4, mlp=O.moe_mlp(6, 2, 8, groups=(3, 2), scale=1.5, shared_ff=8)),
        O.lightning_layer(2, 8, 8, [0.8, 0.9]),
    ], vocab=20, width=16, loop=loop, embed_scale=2.0, logit_scale=0.5)


def test_registry_and_parameter_names():
    from mlx_parallm_b200.utils import _get_classes
    cfg = cfg_small(loop=(0, 2, 2))
    Model, Args = _get_classes(cfg)
    m = Model(Args.from_dict(cfg))
    assert m.model_type == "nifalorn" and m.block_style == "prenorm" and m.supports_ragged and m.dense
    assert sorted(m.parameter_names()) == sorted(O.random_weights(cfg).keys())
    assert m.logit_scale == 0.5 and m.embed.scale == 2.0
    assert m.runs[0].norm2_w_name == "l0.norm2" and m.runs[-1].norm2_w_name is None      # the last layer has no feed-forward


@pytest.mark.parametrize("loop,want", [
    (None, [0, 1, 2]),
    ((0, 2, 2), [0, 1, 0, 1, 2]),
    ((1, 3, 3), [0, 1, 2, 1, 2, 1, 2]),
    ((1, 2, 1), [0, 1, 2]),
    ((2, 2, 4), [0, 1, 2]),
    ((0, 3, 2), [0, 1, 2, 0, 1, 2]),
])
def test_run_order_of_a_looped_span(loop, want):
    from mlx_parallm_b200.utils import _get_classes
    cfg = cfg_small(loop=loop)
    assert O.layer_runs(cfg) == want
    Model, Args = _get_classes(cfg)
    m = Model(Args.from_dict(cfg))
    assert [r.layer for r in m.runs] == want
    assert [r.slot for r in m.runs] == list(range(len(want)))            # one state per run, also for a layer that runs again
    assert not any(r.opens for r in m.runs) and m.loop_in is None           # nothing happens between passes
    for r in m.runs:
        assert r.mixer is m.mixers[r.layer]                                # the same modules (weights) every pass


def test_config_checks():
    from mlx_parallm_b200.utils import _get_classes
    cfg = cfg_small()
    Model, Args = _get_classes(cfg)
    with pytest.raises(NotImplementedError):
        Args.from_dict(dict(cfg, layers=[dict(cfg["layers"][0], type="delta")]))
    with pytest.raises(NotImplementedError):
        Args.from_dict(dict(cfg, layers=[dict(cfg["layers"][0], mlp={"kind": "sparse"})]))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, loop={"start": 2, "stop": 5, "times": 2}))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, layers=[O.attention_layer(3, 2, 8, 8, 0.3, 0.4, 5, 4)]))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, layers=[O.ssm_layer(3, 8, 6, 2, 1, conv=2)]))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, layers=[O.lightning_layer(3, 8, 8, [0.5, 0.6])]))
    with pytest.raises(ValueError):                                          # two kept groups of two experts cannot give five
        Args.from_dict(dict(cfg, layers=[O.lightning_layer(1, 8, 8, [0.5], mlp=O.moe_mlp(6, 5, 8, groups=(3, 2)))]))


@pytest.mark.parametrize("dims,base,scaling", [(8, 10000.0, None), (16, 5e5, (4.0, 1.0, 8.0, 2048)), (32, 500000.0, (8.0, 1.0, 4.0, 8192)),
                                                (6, 100.0, (2.0, 1.0, 8.0, 64))])
def test_rotation_rates(dims, base, scaling):
    from mlx_parallm_b200.models._sequence import rotary_rates
    rot = {"dims": dims, "base": base}
    sc = None
    if scaling:
        sc = rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    got = rotary_rates(dims, base, sc)
    want = O.rotation_rates(rot).tolist()
    assert len(got) == dims // 2 and all(abs(a - b) <= 1e-12 * abs(b) for a, b in zip(got, want))
    if scaling:
        plain = rotary_rates(dims, base)
        kinds = {"kept": 0, "slowed": 0, "blended": 0}
        for f, g in zip(plain, got):
            l = 2 * math.pi / f
            if l < sc["original"] / sc["high"]:
                assert g == f
                kinds["kept"] += 1
            elif l > sc["original"] / sc["low"]:
                assert abs(g - f / sc["factor"]) < 1e-15
                kinds["slowed"] += 1
            else:
                assert f / sc["factor"] < g < f
                kinds["blended"] += 1
        assert kinds["kept"] and kinds["slowed"]


def test_oracle_prefix_property_chunks_and_groups():
    """The oracle is causal (a prefix gives the prefix's logits), its attention forgets at a chunk's border, and its router
    never picks from a dropped group: these hold for any correct statement of the design and guard the oracle itself."""
    cfg = cfg_small(loop=(0, 2, 2))
    w = O.random_weights(cfg, 1)
    t = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    full = O.forward(cfg, w, t)
    assert (O.forward(cfg, w, t[:6]) - full[:6]).abs().max() < 1e-9
    P = {k: v.double() for k, v in w.items()}
    m = cfg["layers"][1]["mixer"]
    h = torch.randn(12, 16, dtype=O.F64)
    a = O.differential_attention(h, P, "l1.mix.", m, 1e-5)
    h2 = h.clone()
    h2[:5] = torch.randn(5, 16, dtype=O.F64)                                # the first chunk (5 positions) changes
    b = O.differential_attention(h2, P, "l1.mix.", m, 1e-5)
    assert (a[5:] - b[5:]).abs().max() < 1e-12 and (a[:5] - b[:5]).abs().max() > 1e-3
    r = cfg["layers"][1]["mlp"]["router"]
    P["l1.mlp.correction"] = torch.tensor([-5.0, -5.0, 0.0, 0.0, -4.0, -4.5], dtype=O.F64)   # negative picking scores everywhere but group 1
    ids, wts = O.route(h, P, "l1.mlp.", r)
    assert set(ids.flatten().tolist()) <= {2, 3, 4, 5}                      # group 0 is dropped although its scores beat -inf
    assert (wts.sum(-1) - r["scale"]).abs().max() < 1e-9
