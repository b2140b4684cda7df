"""The Nufolix configuration on the CPU: keys, the parts it names, tensor names and shapes, what each layer asks of the
cache manager, refusals, and the plain implementation's own consistency (a sequence's logits do not depend on what
follows; the recurrences agree with their closed forms on inputs made for that)."""

import copy

import pytest
import torch

import nufolix_cases as N
import plain_nufolix as plain


def test_the_specification_names_every_tensor_the_plain_implementation_reads():
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.models import build_model

    for name, cfg in N.CONFIGS.items():
        config = resolve_config(cfg)
        model = build_model(config)
        expected = {n: tuple(s.shape) for n, s in model.expected_params().items() if not s.optional}
        W = N.weights_for(cfg, 0)
        got = {n: tuple(t.shape) for n, t in W.items()}
        # the inner sizes of the two-step projections are the tensors' to give
        loose = {n: tuple(None if x is None else x for x in s) for n, s in expected.items()}
        assert set(loose) == set(got), name
        for n, shape in loose.items():
            assert len(shape) == len(got[n]) and all(a is None or a == b for a, b in zip(shape, got[n])), (name, n, shape, got[n])
        plain.forward(cfg, {k: v.double() for k, v in W.items()}, [1, 2, 3])       # and the oracle needs no other
        assert config.to_json()["layers"] == cfg["layers"]
        assert resolve_config(config.to_json()).model_spec() == config.model_spec()
        assert config.parameter_counts()["total_parameters"] > 0


def test_what_the_layers_ask_of_the_cache_manager():
    from llm_pipeline_b200.cache import HeadRowPagesSpec
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.models import build_model

    cfg = N.CONFIGS["mixed"]
    model = build_model(resolve_config(cfg))
    specs = model.cache_specs()
    assert len(specs) == 4
    # a state-space layer keeps no pages: two copies of its last taps - 1 inputs and of its state
    m = cfg["layers"][0]["mixer"]
    channels = m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
    pages, state = specs[0]
    assert pages is None and state.shape == (2 * (m["conv"] - 1) * channels + 2 * m["heads"] * m["state"] * m["vdim"],)
    assert state.dtype == torch.float32
    # a parallel layer: pages of [key | value] rows for the left mixer, a float32 state for the right one
    l, r = cfg["layers"][1]["mixer"]["left"], cfg["layers"][1]["mixer"]["right"]
    pages, state = specs[1]
    assert pages == HeadRowPagesSpec(l["kv_heads"], l["dim"] + l["vdim"], None)
    channels = 2 * r["kv_heads"] * r["dim"] + r["heads"] * r["vdim"]
    assert state.shape == (2 * (r["conv"] - 1) * channels + 2 * r["heads"] * r["dim"] * r["vdim"],) and state.dtype == torch.float32
    assert model.blocks[1].feed_forward is None and model.blocks[0].feed_forward is not None


@pytest.mark.parametrize("damage, message", [
    (lambda c: c["layers"][0].update(type="lstm"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].pop("state"), "lacks"),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("conv"), "lacks"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "lacks"),
    (lambda c: c["layers"][0]["mixer"].update(groups=3), "cannot share"),
    (lambda c: c["layers"][0]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "cannot share"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown mlp kind"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "needs ff"),
    (lambda c: c.pop("norm"), "required keys"),
    (lambda c: c.update(layers=[]), "required keys|no layers"),
])
def test_refusals(damage, message):
    from llm_pipeline_b200.config import resolve_config

    cfg = copy.deepcopy(N.CONFIGS["mixed"])
    damage(cfg)
    with pytest.raises(ValueError, match=message):
        resolve_config(cfg)


def test_defaults_where_the_configuration_is_silent():
    from llm_pipeline_b200.config import resolve_config

    cfg = copy.deepcopy(N.CONFIGS["mixed"])
    cfg.pop("residual_mult")
    cfg.pop("embedding")
    config = resolve_config(cfg)
    assert config.residual_mult == 1.0 and config.embedding_scale == 1.0
    spec = config.model_spec()
    assert spec.layers[3].mixer.args["left"]["args"]["softcap"] is None and spec.layers[3].mixer.args["left"]["args"]["position"] is None
    assert spec.layers[1].mixer.args["left"]["args"]["rotary_dim"] == 8


def test_the_plain_implementation_is_causal_and_its_recurrences_have_their_closed_forms():
    cfg = N.CONFIGS["mixed"]
    W = {k: v.double() for k, v in N.weights_for(cfg, 1).items()}
    tokens = list(range(3, 40))
    whole = plain.forward(cfg, W, tokens)
    assert (plain.forward(cfg, W, tokens[:17]) - whole[:17]).abs().max() < 1e-9
    # a convolution whose taps are (0, .., 0, 1) is the identity, and one whose first tap alone is 1 is a shift by taps - 1
    x = torch.randn(9, 5, dtype=torch.float64)
    taps = torch.zeros(5, 4, dtype=torch.float64)
    taps[:, -1] = 1
    assert torch.equal(plain.short_convolution(x, taps), x)
    taps = torch.zeros(5, 4, dtype=torch.float64)
    taps[:, 0] = 1
    assert torch.equal(plain.short_convolution(x, taps)[3:], x[:-3]) and plain.short_convolution(x, taps)[:3].abs().max() == 0
    # the activation is continuous with slope 1/2 at zero, whatever its two numbers are
    act = torch.tensor([0.3, -1.2], dtype=torch.float64)
    e = 1e-6
    lo, hi = plain.xielu(torch.tensor([-e], dtype=torch.float64), act), plain.xielu(torch.tensor([e], dtype=torch.float64), act)
    assert abs(float(hi - lo) / (2 * e) - 0.5) < 1e-4 and abs(float(hi + lo)) < 1e-9
    # a rotation keeps lengths, leaves the entries past its size alone and turns a pair by position * frequency
    v = torch.randn(6, 2, 12, dtype=torch.float64)
    r = plain.rotate_half(v, torch.arange(6), 8, 100.0)
    assert torch.equal(r[..., 8:], v[..., 8:]) and (r.norm(dim=-1) - v.norm(dim=-1)).abs().max() < 1e-12
    assert torch.equal(r[0], v[0])
    one = torch.zeros(1, 1, 8, dtype=torch.float64)
    one[0, 0, 1] = 1.0                                                   # pair (1, 5), frequency 100^(-2/8)
    a = 7 * 100.0 ** (-2.0 / 8)
    turned = plain.rotate_half(one, torch.tensor([7]), 8, 100.0)[0, 0]
    assert abs(float(turned[1]) - torch.cos(torch.tensor(a, dtype=torch.float64))) < 1e-12
    assert abs(float(turned[5]) - torch.sin(torch.tensor(a, dtype=torch.float64))) < 1e-12
