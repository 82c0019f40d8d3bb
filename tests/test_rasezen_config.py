"""Rasezen's configuration without a GPU: parsing, the model's description as data, refusals."""
import copy
import json

import pytest
import torch

from rasezen_models import SMALL, make_weights, write_model


def test_round_trip_and_spec():
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.config.rasezen import RasezenConfig
    for name, d in SMALL.items():
        cfg = config_from_dict(d)
        assert isinstance(cfg, RasezenConfig)
        assert cfg.to_dict() == d, name
        assert config_from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
        spec = cfg.model_spec()
        assert [l.block for l in spec.layers] == ["parallel"] * len(d["layers"])
        assert [l.mixer.kind for l in spec.layers] == [
            "mamba2" if L["type"] == "mamba2" else "wide_norm_attention" for L in d["layers"]]
        kinds = {None: None, "dense": "xielu_mlp", "moe": "routed_experts"}
        assert [None if l.ffn is None else l.ffn.kind for l in spec.layers] == [
            kinds[None if L["mlp"] is None else L["mlp"]["kind"]] for L in d["layers"]]
        assert spec.final_norm.params["scalar"] and spec.head.params["tensor"] == "head"


def test_expected_tensors_are_the_designs_names():
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.engine.model import expected_tensors
    for name, d in SMALL.items():
        exp = expected_tensors(config_from_dict(d).model_spec())
        made = make_weights(d, 0)
        assert set(exp) == set(made), (name, set(exp) ^ set(made))
        for n, (shape, _) in exp.items():
            assert tuple(made[n].shape) == tuple(shape), n


def test_sizes_are_read_layer_by_layer():
    from lumenllm_b200.config import config_from_dict
    spec = config_from_dict(SMALL["X"]).model_spec()
    a, s = spec.layers[0].mixer.params, spec.layers[1].mixer.params
    assert (a["num_heads"], a["num_kv_heads"], a["head_dim"], a["value_dim"], a["window"]) == (4, 2, 16, 24, 9)
    assert a["position"].params["rotary_dim"] == 8 and a["value_norm"]
    assert (s["num_heads"], s["head_dim"], s["state_size"], s["groups"], s["taps"], s["norm_groups"]) == (4, 16, 8, 1, 4, 1)
    f = spec.layers[1].ffn.params
    assert (f["num_experts"], f["identity_experts"], f["top"], f["scale"], f["shared_size"]) == (4, 1, 2, 1.5, 32)
    assert spec.layers[2].ffn is None
    y = config_from_dict(SMALL["Y"]).model_spec()
    assert y.layers[2].mixer.params["position"].kind == "none" and y.layers[2].mixer.params["window"] == 0


@pytest.mark.parametrize("edit, words", [
    (lambda d: d["layers"][0].update(type="conv"), "not a mixer"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][1]["mixer"].update(groups=3), "not a multiple"),
    (lambda d: d["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda d: d["layers"][1]["mlp"].update(kind="glu"), "not a feed-forward"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda d: d.pop("norm"), "missing key"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
])
def test_refusals(edit, words):
    from lumenllm_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(SMALL["X"])
    edit(d)
    with pytest.raises(ConfigError, match=words):
        config_from_dict(d)


def test_a_written_model_is_found_by_its_architecture(tmp_path):
    from lumenllm_b200.config import load_config
    from lumenllm_b200.weights.loader import check_against, open_checkpoint
    from lumenllm_b200.engine.model import expected_tensors
    folder = write_model(SMALL["Y"], tmp_path / "m", seed=3)
    cfg = load_config(folder)
    exp = {n: s for n, (s, _) in expected_tensors(cfg.model_spec()).items()}
    assert check_against(exp, open_checkpoint(folder)) == ([], {})
    assert open_checkpoint(folder)["final.norm"].shape == ()


def test_plain_pieces_against_their_definitions():
    """The oracle's own pieces on values worked out by hand."""
    import math
    import plain_rasezen as P
    z = torch.tensor([-2.0, 0.0, 1.5])
    p, q = torch.tensor(0.3), torch.tensor(-0.2)
    sp = lambda v: math.log1p(math.exp(v))
    want = [(0.5 + sp(-0.2)) * (math.exp(-2.0) - 1 + 2.0) - 1.0, 0.0, sp(0.3) * 2.25 + 0.75]
    assert torch.allclose(P.xielu(z, p, q), torch.tensor(want), atol=1e-6)
    x = torch.arange(6.0).view(1, 1, 6)
    r = P.rotate(x, torch.tensor([2]), 100.0, 4)
    a0, a1 = 2.0, 2.0 / 10.0
    want = [0 * math.cos(a0) - 2 * math.sin(a0), 1 * math.cos(a1) - 3 * math.sin(a1),
            2 * math.cos(a0) + 0 * math.sin(a0), 3 * math.cos(a1) + 1 * math.sin(a1), 4.0, 5.0]
    assert torch.allclose(r.view(-1), torch.tensor(want), atol=1e-5)
    assert P.window_mask(5, 2).int().tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 1, 1, 0, 0], [0, 0, 1, 1, 0],
                                                  [0, 0, 0, 1, 1]]
    c = P.causal_conv(torch.tensor([[1.0], [2.0], [4.0]]), torch.tensor([[10.0, 1.0]]), torch.tensor([0.5]))
    assert c.view(-1).tolist() == [1.5, 12.5, 24.5]
