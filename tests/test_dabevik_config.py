"""Dabevik without a GPU: config.json to typed configuration and back, what is refused, the
model's parts as data (layers that share tensors, a layer without feed-forward), the names and
shapes of its tensors, and the cache's bookkeeping for a window that keeps first tokens."""
import copy

import pytest

from dabevik_models import SMALL, make_weights


def test_round_trip_and_registry():
    from lumenllm_b200.config import DabevikConfig, config_from_dict
    for name, d in SMALL.items():
        c = config_from_dict(d)
        assert isinstance(c, DabevikConfig)
        assert c.to_dict() == d
        assert config_from_dict(c.to_dict()) == c


def test_layers_that_share_tensors_become_schedule_entries():
    from lumenllm_b200.config import config_from_dict
    spec = config_from_dict(SMALL["X"]).model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 0]            # layer 2 runs layer 0's tensors
    assert len(spec.layers) == 2 and spec.layers[1].ffn is None
    assert spec.layers[0].block == "sandwich_conv" and spec.layers[0].mixer.kind == "talking_attention"
    spec = config_from_dict(SMALL["Z"]).model_spec()
    assert [e.layer for e in spec.schedule] == [0, 1, 1]
    p = spec.layers[1].mixer.params
    assert (p["num_heads"], p["num_kv_heads"], p["head_dim"], p["value_dim"], p["window"], p["keep_first"]) == \
        (2, 2, 64, 128, 33, 70)
    chain = copy.deepcopy(SMALL["X"])
    chain["layers"].append(dict(chain["layers"][2], weights_of=2))   # a layer that names a layer that names one
    assert [e.layer for e in config_from_dict(chain).model_spec().schedule] == [0, 1, 0, 0]


def test_expected_tensors_are_the_designs_names():
    from lumenllm_b200.config import config_from_dict
    from lumenllm_b200.engine.model import expected_tensors
    for name, d in SMALL.items():
        want = {k: tuple(v.shape) for k, v in make_weights(d, 0).items()}
        got = {k: tuple(shape) for k, (shape, _) in expected_tensors(config_from_dict(d).model_spec()).items()}
        assert got == want, name


@pytest.mark.parametrize("edit, word", [
    (lambda d: d.pop("canon"), "canon"),
    (lambda d: d["layers"][0].update(type="recurrent"), "type"),
    (lambda d: d["layers"][1].update(mixer=dict(d["layers"][1]["mixer"], kv_heads=3)), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["mask"].pop("size"), "size"),
    (lambda d: d["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "dense"),
    (lambda d: d["layers"][2].update(weights_of=7), "weights_of"),
    (lambda d: d["layers"][2].update(mixer=dict(d["layers"][2]["mixer"], dim=8)), "other sizes"),
    (lambda d: d["embedding"].update(scale="big"), "scale"),
])
def test_what_is_refused(edit, word):
    from lumenllm_b200.config import ConfigError, config_from_dict
    d = copy.deepcopy(SMALL["X"])
    edit(d)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_pages_of_kept_first_tokens_stay_while_the_window_moves():
    from lumenllm_b200.cache import PAGE, CacheNeed, KVCache
    need = CacheNeed(2, 16, window=PAGE + 10, v_dim=24, keep_first=PAGE + 3)     # two pages of kept tokens
    cache = KVCache({0: need, 1: CacheNeed(2, 16)}, 16 * PAGE, 2, 16 * PAGE)
    windowed = cache.groups[cache.group_of[0]]
    everything = cache.groups[cache.group_of[1]]
    assert windowed.need.value_dim == 24 and everything.need.value_dim == 16
    s = cache.alloc_slot()
    for step in range(10 * PAGE):
        cache.reserve(s, 1)
        cache.commit(s, 1)
        n = step + 1
        held = {i for i in range(windowed.table.shape[1]) if windowed.table[s, i] != 0}
        first_seen = max(0, n - need.window + 1) // PAGE
        want = set(range(min(2, -(-n // PAGE)))) | set(range(first_seen, -(-n // PAGE)))
        assert held == want, (n, held, want)
        assert int(windowed.n_held[s]) == len(held)
        assert int(everything.n_held[s]) == -(-n // PAGE)
    cache.check()
    cache.free_slot(s)
    cache.check()
    assert windowed.pool.free_count == everything.pool.free_count == 16
    s = cache.alloc_slot()                       # the slot and its pages once more
    cache.reserve(s, 3 * PAGE)
    cache.commit(s, 3 * PAGE)
    assert int(windowed.n_held[s]) == 3 and windowed.table[s, 0] != 0
    cache.check()
