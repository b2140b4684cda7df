"""The Tupidra configuration on the CPU: keys, the parts it names, tensor names and shapes, what each layer asks of the
cache manager (pages, kept first tokens, state, rows read from another layer), refusals, the frequency ramp, and the
plain implementation's own consistency."""

import copy
import math

import pytest
import torch

import plain_tupidra as plain
import tupidra_cases as T


def test_the_specification_names_every_tensor_the_plain_implementation_reads():
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.models import build_model

    for name, cfg in T.CONFIGS.items():
        config = resolve_config(cfg)
        model = build_model(config)
        expected = {n: tuple(s.shape) for n, s in model.expected_params().items() if not s.optional}
        W = T.weights_for(cfg, 0)
        assert expected == {n: tuple(t.shape) for n, t in W.items()}, name
        plain.forward(cfg, {k: v.double() for k, v in W.items()}, [1, 2, 3])       # and the oracle needs no other
        assert config.to_json()["layers"] == cfg["layers"]
        assert resolve_config(config.to_json()).model_spec() == config.model_spec()
        assert config.parameter_counts()["total_parameters"] > 0
        # a layer without a feed-forward may still find its second norm and filter in a checkpoint, and reads neither
        spare = {n for n, s in model.expected_params().items() if s.optional}
        bare = [i for i, layer in enumerate(cfg["layers"]) if layer["mlp"] is None]
        assert spare == {f"l{i}.norm2" for i in bare} | ({f"l{i}.canon2" for i in bare} if cfg["canon"]["taps"] else set())


def test_what_the_layers_ask_of_the_cache_manager():
    from llm_pipeline_b200.cache import CacheManager
    from llm_pipeline_b200.cache.spec import HeadRowPagesSpec, TokenPagesSpec
    from llm_pipeline_b200.config import resolve_config
    from llm_pipeline_b200.models import build_model

    cfg = T.CONFIGS["mixed"]
    model = build_model(resolve_config(cfg))
    specs = model.cache_specs()
    D, taps = cfg["width"], cfg["canon"]["taps"]
    assert len(specs) == 6
    filters = lambda sublayers: 2 * (taps - 1) * D * sublayers      # noqa: E731  two copies of the last taps - 1 inputs
    m = cfg["layers"][0]["mixer"]
    pages, state = specs[0]
    assert pages is None and state.dtype == torch.float32
    assert state.shape == (filters(2) + 2 * (m["conv"] - 1) * m["inner"] + 2 * m["inner"] * m["state"],)
    a = cfg["layers"][1]["mixer"]
    assert specs[1] == (HeadRowPagesSpec(a["kv_heads"], a["dim"] + a["vdim"], 40, 3), specs[1][1]) and specs[1][1].shape == (filters(2),)
    l = cfg["layers"][2]["mixer"]
    assert specs[2][0] == TokenPagesSpec((l["kv_rank"] + l["rot_dim"],), None) and specs[2][1].shape == (filters(2),)
    assert specs[3][0] is None and specs[3][1].shape[0] > filters(1)            # a layer without feed-forward filters one input
    assert specs[4][0] == HeadRowPagesSpec(3, 48, None, 0)
    # the layer that reads another layer's rows keeps no pages, only its filters' inputs; its execution names the other cache
    assert specs[5][0] is None and specs[5][1].shape == (filters(1),)
    assert [e.pages_from for e in model.spec.schedule] == [None, None, None, None, None, 2]
    assert "l5.mix.dkv" not in model.expected_params() and "l2.mix.dkv" in model.expected_params()
    # a windowed group gives pages back as the window passes them, but for those of the kept first tokens
    cache = CacheManager(specs, page_size=4, num_pages=64, max_requests=2, max_request_tokens=128)
    windowed = [g for g, group in enumerate(cache.groups) if group.spec.window == 40][0]
    cache.admit("a")
    assert cache.reserve("a", 100)
    cache.commit("a", 100)
    table = cache.block_table("a", windowed)
    assert table[0] >= 0 and all(p < 0 for p in table[1:15]) and all(p >= 0 for p in table[15:25])
    cache.check()
    cache.free("a")
    cache.check()


@pytest.mark.parametrize("damage, message", [
    (lambda c: c["layers"][0].update(type="lstm"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].pop("state"), "lacks"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "lacks"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "lacks"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "cannot share"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][5]["mixer"].update(kv_from=4), "kv_from"),
    (lambda c: c["layers"][5]["mixer"].update(kv_from=5), "kv_from"),
    (lambda c: c["layers"][5]["mixer"].update(kv_rank=48), "must equal"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "unknown mlp kind"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "needs ff"),
    (lambda c: c.pop("norm"), "required keys"),
    (lambda c: c.update(layers=[]), "required keys|no layers"),
])
def test_refusals(damage, message):
    from llm_pipeline_b200.config import resolve_config

    cfg = copy.deepcopy(T.CONFIGS["mixed"])
    damage(cfg)
    with pytest.raises(ValueError, match=message):
        resolve_config(cfg)


def test_defaults_where_the_configuration_is_silent():
    from llm_pipeline_b200.config import resolve_config

    cfg = copy.deepcopy(T.CONFIGS["mixed"])
    cfg.pop("canon")
    spec = resolve_config(cfg).model_spec()
    assert all(not layer.block_args for layer in spec.layers)                      # no filters in front of the sublayers
    assert spec.layers[4].mixer.args["window"] is None and spec.layers[4].mixer.args["softcap"] is None
    assert spec.layers[1].mixer.args["keep_first"] == 3 and spec.layers[1].mixer.args["window"] == 40
    cfg["layers"][2]["mixer"]["rot"].pop("scaling")
    cfg["layers"][5]["mixer"]["rot"].pop("scaling")
    spec = resolve_config(cfg).model_spec()
    (only,) = spec.positions.values()
    assert only.args["scaling"] == 1.0 and "frequency_scaling" not in only.args


def test_the_frequency_ramp_of_the_rotation():
    from llm_pipeline_b200.parts.position import RotaryPositions

    for dims, base, rule in ((8, 100.0, T.RAMP), (32, 50000.0, {"factor": 4.0, "original": 128, "fast": 8.0, "slow": 1.0}),
                             (6, 37.0, {"factor": 3.0, "original": 20, "fast": 4.0, "slow": 1.0})):
        want, magnitude = plain.yarn_frequencies(dims, base, rule)
        got = RotaryPositions.ramp_frequencies(dims, base, dict(rule, kind="ramp"))
        assert torch.allclose(torch.tensor(got, dtype=torch.float64), want, rtol=1e-12, atol=0)
        assert magnitude == 0.1 * math.log(rule["factor"]) + 1.0
    ramp, _ = plain.yarn_frequencies(8, 100.0, T.RAMP)
    plain_f, _ = plain.yarn_frequencies(8, 100.0, None)
    assert ramp[0] == plain_f[0] and abs(float(ramp[1] / plain_f[1]) - (0.5 / 8 + 0.5)) < 1e-12 and abs(float(ramp[3] / plain_f[3]) - 1 / 8) < 1e-12


def test_the_plain_implementation_is_causal_and_its_mechanisms_have_their_closed_forms():
    cfg = T.CONFIGS["mixed"]
    W = {k: v.double() for k, v in T.weights_for(cfg, 1).items()}
    tokens = list(range(3, 70))
    whole = plain.forward(cfg, W, tokens)
    assert (plain.forward(cfg, W, tokens[:17]) - whole[:17]).abs().max() < 1e-9
    # an input filter with zero taps is the identity; with the last tap alone it doubles; the first tap alone adds a shift
    x = torch.randn(9, 5, dtype=torch.float64)
    taps = torch.zeros(5, 4, dtype=torch.float64)
    assert torch.equal(plain.input_conv(x, taps), x)
    taps[:, 0] = 1
    assert torch.equal(plain.input_conv(x, taps)[3:], x[3:] + x[:-3]) and torch.equal(plain.input_conv(x, taps)[:3], x[:3])
    # the interleaved rotation keeps lengths (times the magnitude), leaves the entries past its size alone and turns pair (2, 3)
    v = torch.randn(6, 2, 12, dtype=torch.float64)
    r = plain.rotate_interleaved(v, torch.arange(6), 8, 100.0, None)
    assert torch.equal(r[..., 8:], v[..., 8:]) and (r.norm(dim=-1) - v.norm(dim=-1)).abs().max() < 1e-12 and torch.equal(r[0], v[0])
    one = torch.zeros(1, 1, 8, dtype=torch.float64)
    one[0, 0, 2] = 1.0
    a = 7 * 100.0 ** (-2.0 / 8)
    turned = plain.rotate_interleaved(one, torch.tensor([7]), 8, 100.0, None)[0, 0]
    assert abs(float(turned[2]) - math.cos(a)) < 1e-12 and abs(float(turned[3]) - math.sin(a)) < 1e-12
    # window attention: with one key in sight and a zero score the sink takes half; a kept first token stays in sight
    q, k, val = torch.zeros(12, 2, 4, dtype=torch.float64), torch.zeros(12, 1, 4, dtype=torch.float64), torch.ones(12, 1, 3, dtype=torch.float64)
    out = plain.attend_window(q, k, val, 1.0, None, 1, 0)
    assert torch.allclose(out, torch.full_like(out, 0.5))
    val[0] = 100.0
    far = plain.attend_window(q, k, val, 1.0, None, 2, 1)[11]
    gone = plain.attend_window(q, k, val, 1.0, None, 2, 0)[11]
    near = [math.exp(-2.0 ** (-8.0 * (h + 1) / 2)) for h in range(2)]            # the key one token back lost its head's slope
    assert float(far.max()) > 1.0 and all(abs(float(gone[h, 0]) - (1.0 + near[h]) / (2.0 + near[h])) < 1e-12 for h in range(2))
    # the scan with a zero decay rate is a running sum; a state handed on gives the same rows as the whole sequence
    x, dt = torch.randn(7, 3, dtype=torch.float64), torch.rand(7, 3, dtype=torch.float64)
    B, C = torch.randn(7, 2, dtype=torch.float64), torch.randn(7, 2, dtype=torch.float64)
    y, _ = plain.scan(x, dt, torch.zeros(3, 2, dtype=torch.float64), B, C, torch.zeros(3, dtype=torch.float64))
    running = torch.cumsum((dt * x)[:, :, None] * B[:, None, :], dim=0)
    assert torch.allclose(y, torch.einsum("tcn,tn->tc", running, C))
    A = -torch.rand(3, 2, dtype=torch.float64)
    whole_y, _ = plain.scan(x, dt, A, B, C, torch.ones(3, dtype=torch.float64))
    head, S = plain.scan(x[:4], dt[:4], A, B[:4], C[:4], torch.ones(3, dtype=torch.float64))
    tail, _ = plain.scan(x[4:], dt[4:], A, B[4:], C[4:], torch.ones(3, dtype=torch.float64), S)
    assert torch.allclose(torch.cat([head, tail]), whole_y)


def test_a_random_model_folder_can_be_written_and_read_back(tmp_path):
    from llm_pipeline_b200.config import load_config
    from llm_pipeline_b200.models import build_model
    from llm_pipeline_b200.weights import write_random_model
    from llm_pipeline_b200.weights.source import SafetensorsSource, check_names_and_shapes

    folder = write_random_model(T.CONFIGS["mixed"], 3, str(tmp_path))
    config = load_config(folder)
    assert config.architecture == "Tupidra"
    source = SafetensorsSource(folder)
    check_names_and_shapes(build_model(config).expected_params(), source)
    assert abs(float(source.get("l0.norm1").float().mean()) - 1.0) < 0.3          # around one, not noise around zero
    assert source.shape("l5.mix.uq") == (2 * (24 + 8), 12) and "l5.mix.dkv" not in source.names()
    source.close()
