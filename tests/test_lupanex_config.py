"""Lupanex on the CPU: the configuration reader, the manifest, the order of runs, and the plain implementation's own pieces."""
import copy
import math

import numpy as np
import pytest

import lupanex_models as LM
import plain_lupanex as PL
from vitna_anchor_b200.config import ConfigError, LupanexConfig, resolve
from vitna_anchor_b200.models.lupanex import lupanex_manifest
from vitna_anchor_b200.parts.attention import distance_bucket


@pytest.mark.parametrize("name", sorted(LM.CONFIGS))
def test_config_reads_back_and_names_every_tensor(name):
    cj = LM.CONFIGS[name]
    arch = resolve(cj)
    assert arch.name == "Lupanex"
    cfg = arch.parse_config(cj)
    assert LupanexConfig.from_dict(cfg.to_dict()) == cfg
    made = LM.make_tensors(cj, 0, LM.REL_ROWS[name])
    specs = {w.name: w for w in lupanex_manifest(cfg)}
    assert set(specs) == set(made)
    for n, t in made.items():
        assert specs[n].fits(t.shape), n
    assert cfg.runs() == PL.layer_order(cj)


def test_the_order_of_runs():
    cj = copy.deepcopy(LM.CONFIGS["plain"])
    assert LupanexConfig.from_dict(cj).runs() == [0, 1, 2, 3]
    cj["loop"] = dict(start=1, stop=3, times=3)
    assert LupanexConfig.from_dict(cj).runs() == [0, 1, 2, 1, 2, 1, 2, 3]
    cj["loop"] = dict(start=3, stop=4, times=2)
    assert LupanexConfig.from_dict(cj).runs() == [0, 1, 2, 3, 3]
    cj["loop"] = dict(start=2, stop=2, times=5)                  # an empty range runs nothing twice
    assert LupanexConfig.from_dict(cj).runs() == [0, 1, 2, 3]


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(window=7), "window"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mlp"].update(kind="experts"), "kind"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3, kv_heads=2), "kv_heads"),
    (lambda c: c.update(loop=dict(start=3, stop=9, times=2)), "loop"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_what_the_engine_does_not_have_is_refused_by_name(change, word):
    cj = copy.deepcopy(LM.CONFIGS["plain"])
    change(cj)
    with pytest.raises(ConfigError, match=word):
        LupanexConfig.from_dict(cj)


def test_sizes_that_may_be_left_out():
    cj = copy.deepcopy(LM.CONFIGS["plain"])
    del cj["layers"][1]["mixer"]["kv_heads"], cj["layers"][1]["mixer"]["vdim"]
    m = LupanexConfig.from_dict(cj).layers[1].mixer
    assert (m.kv_heads, m.vdim) == (m.heads, m.dim)


def test_distance_buckets():
    for rows, far in ((16, 100), (12, 40), (6, 9), (32, 128), (8, 512)):
        half = rows // 2
        b = [distance_bucket(n, rows, far) for n in range(3 * far)]
        assert b == [PL.distance_bucket(n, rows, far) for n in range(3 * far)]
        assert b[:half] == list(range(half)) and b[half] == half
        assert all(x <= y for x, y in zip(b, b[1:])) and b[far] == rows - 1 and max(b) == rows - 1
        # written out once more: the first distance of every row beyond the exact ones
        for r in range(half, rows):
            first = b.index(r) if r in b else None
            if first is not None:
                assert first >= half * (far / half) ** ((r - half) / (rows - half)) - 1e-9
                assert first - 1 < half * (far / half) ** ((r - half) / (rows - half)) or first == half


def test_the_plain_pieces():
    x = np.linspace(-4, 4, 9)
    assert np.allclose(PL.gelu_erf(x), [0.5 * v * (1 + math.erf(v / math.sqrt(2))) for v in x])
    assert abs(PL.gelu_tanh(np.array([1.0]))[0] - 0.841192) < 1e-6
    assert np.allclose(PL.softplus(np.array([-50.0, 0.0, 50.0])), [0.0, math.log(2), 50.0])
    y = PL.short_conv(np.arange(1.0, 6.0)[:, None], np.array([[100.0, 10.0, 1.0]]))
    assert np.allclose(y[:, 0], [1, 12, 123, 234, 345])          # the last tap is the current token's, zeros before the start
    v = np.array([[3.0, 4.0]])
    assert np.allclose(PL.rms(v, 0.0), v / math.sqrt(12.5))
