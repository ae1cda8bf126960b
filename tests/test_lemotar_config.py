"""The Lemotar configuration on the CPU: the reader of its keys, what it refuses, the model it describes, and the
frequencies of its stretched rotation."""

import copy
import math

import pytest
import torch

from lemotar_tools import CONFIGS, clean
from quantinfer_b200.config import LemotarConfig, RotarySpec, config_from_dict
from quantinfer_b200.engine.model import tensor_needs_of_spec
from quantinfer_b200.errors import ConfigError
from quantinfer_b200.parts.position import direct_frequencies


def test_the_registry_finds_the_class_and_the_dictionary_comes_back():
    for name, cfg in CONFIGS.items():
        c = config_from_dict(clean(cfg))
        assert isinstance(c, LemotarConfig)
        assert c.to_dict() == clean(cfg)
        rebuilt = LemotarConfig(**{k: getattr(c, k) for k in ("vocab", "width", "norm_eps", "alpha", "embedding_scale", "layers")})
        assert LemotarConfig.from_dict(rebuilt.to_dict()) == c


def test_the_model_it_describes():
    s = config_from_dict(clean(CONFIGS["P"])).to_model_spec()
    assert [call.layer for call in s.order] == [0, 1, 2, 3]
    assert [(call.cache, call.writes_cache) for call in s.order] == [(0, True), (1, True), (0, False), (2, True)]
    assert s.embedding.scale == 2.5 and s.final_norm.kind == "rmsnorm_one_plus" and s.final_norm.eps == 3e-6
    lat = s.layers[0]
    assert lat.kind == "postnorm" and lat.alpha == 1.7 and lat.ffn.activation == "silu" and lat.ffn.names == ("gate", "up", "down")
    m = lat.mixer
    assert (m.num_heads, m.head_dim, m.rot_dim, m.value_dim, m.kv_rank, m.window, m.sink, m.out_gate, m.shares_latent) == (
        3, 10, 6, 7, 12, 9, True, True, False)
    assert (m.position.rotary_dim, m.position.theta, m.position.pairing, m.position.stretch) == (4, 300.0, "half_split", (3.0, 64.0, 8.0, 1.0))
    assert s.layers[2].mixer.shares_latent and s.layers[2].mixer.window == 13
    par = s.layers[1]
    assert par.ffn is None and par.ffn_norm is None
    l, r = par.mixer.left, par.mixer.right
    assert (l.num_heads, l.num_kv_heads, l.head_dim, l.value_dim, l.window, l.chunk, l.softcap, l.sink, l.values_from_keys, l.qk_norm) == (
        6, 3, 10, 10, 17, None, 4.0, "zero", True, "whole")
    assert (l.position.rotary_dim, l.position.pairing, l.bias, l.out_gate, l.qk_norm_eps) == (4, "interleaved", False, False, 3e-6)
    assert (r.heads, r.kv_heads, r.head_dim, r.value_dim, r.conv_taps, r.norm_eps, r.unit_eps) == (4, 2, 5, 7, 2, 3e-6, 1e-6)
    assert par.mixer.out_norm_names == ("l1.mix.left.out", "l1.mix.right.out") and par.mixer.sum_scale == 0.5
    needs = tensor_needs_of_spec(s)
    assert "l1.norm2" not in needs and "l2.mix.dkv" not in needs and "l1.mix.left.v" not in needs
    assert needs["l1.mix.right.a1"].shape == (None, 44) and needs["l1.mix.right.a2"].shape == (20, None)
    assert needs["l1.mix.right.q"].shape == (10, 44) and needs["l1.mix.right.v.conv"].shape == (28, 2) and needs["l1.mix.right.norm"].shape == (7,)
    assert needs["l1.mix.left.q.norm"].shape == (60,) and needs["l0.mix.g"].shape == (21, 44) and needs["l0.mix.sink"].shape == (3,)
    # without the optional keys: no rotation, no window, no cap, no embedding factor
    p3 = s.layers[3].mixer.left
    assert p3.position is None and p3.window is None and p3.softcap is None
    q = config_from_dict(clean(CONFIGS["Q"])).to_model_spec()
    assert q.embedding.scale == 1.0 and q.layers[1].mixer.window is None and q.layers[1].mixer.position.stretch is None


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].update(type="attention"), "mixers"),
    (lambda d: d["layers"][1]["mixer"]["left"].update(heads=5), "multiple"),
    (lambda d: d["layers"][1]["mixer"]["left"].update(vdim=6), "values are its keys"),
    (lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=3), "even"),
    (lambda d: d["layers"][1]["mixer"]["left"]["rot"].update(dims=12), "within"),
    (lambda d: d["layers"][1]["mixer"]["left"].update(softcap=0.0), "softcap"),
    (lambda d: d["layers"][1]["mixer"]["right"].update(kv_heads=3), "multiple"),
    (lambda d: d["layers"][1]["mixer"]["right"].update(conv=40), "conv"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=8), "within"),
    (lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.5), "factor"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda d: d["layers"][2]["mixer"].update(kv_from=2), "earlier"),
    (lambda d: d["layers"][2]["mixer"].update(kv_from=1), "earlier"),
    (lambda d: d["layers"][2]["mixer"].update(kv_rank=16), "differ"),
    (lambda d: d["layers"][2]["mixer"]["rot"]["scaling"].update(factor=4.0), "differ"),
    (lambda d: d["layers"][0].update(mlp={"kind": "moe"}), "dense"),
    (lambda d: d["norm"].update(eps=0.0), "eps"),
    (lambda d: d.pop("width"), "width"),
])
def test_what_it_refuses(edit, word):
    d = copy.deepcopy(clean(CONFIGS["P"]))
    edit(d)
    with pytest.raises(ConfigError) as err:
        config_from_dict(d)
    assert word in str(err.value)


def test_a_reader_of_a_reader_is_refused():
    d = copy.deepcopy(clean(CONFIGS["Q"]))
    d["layers"].append(copy.deepcopy(d["layers"][2]))
    d["layers"][4]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError) as err:
        config_from_dict(d)
    assert "of its own" in str(err.value)


def test_the_frequencies_of_a_stretched_rotation():
    """Pairs that turn often keep their frequency, pairs that turn seldom have it divided by the factor, a ramp lies
    between; cos and sin grow with the logarithm of the factor."""
    dims, base, factor, original, fast, slow = 16, 1000.0, 4.0, 256.0, 4.0, 1.0
    f, mag = direct_frequencies(RotarySpec(dims, base, "half_split", stretch=(factor, original, fast, slow)))
    plain, one = direct_frequencies(RotarySpec(dims, base, "half_split"))
    assert one == 1.0 and mag == pytest.approx(0.1 * math.log(factor) + 1.0)
    want = []
    lo = max(math.floor(dims * math.log(original / (2 * math.pi * fast)) / (2 * math.log(base))), 0)
    hi = min(math.ceil(dims * math.log(original / (2 * math.pi * slow)) / (2 * math.log(base))), dims - 1)
    for i in range(dims // 2):
        fi = base ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        want.append(fi / factor * ramp + fi * (1.0 - ramp))
    assert torch.allclose(f.double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6)
    assert float(f[0]) == float(plain[0]) and float(f[-1]) == pytest.approx(float(plain[-1]) / factor, rel=1e-6)
    assert lo < hi and 0 < lo       # the premise: the ramp lies inside the pairs


def test_tensors_are_drawn_with_free_ranks():
    from quantinfer_b200.weights import random_weights
    from quantinfer_b200.weights.loader import TensorNeed

    s = config_from_dict(clean(CONFIGS["R"])).to_model_spec()
    needs = tensor_needs_of_spec(s)
    assert needs["l1.mix.right.g1"] == TensorNeed((None, 48)) and needs["l1.mix.right.g2"].drawn_shape() == (48, 16)
    assert hasattr(random_weights, "__name__")


def test_the_comparison_of_the_bench_holds_equal_weights():
    """`bench.py --compare lemotar`: both stacks are valid configurations of their designs and hold the same weights to 3 %."""
    import bench

    for size in bench.LEMOTAR_SIZES:
        new, old = bench.lemotar_entries(size)
        a, b = (bench.model_arithmetic(c, c.to_model_spec()) for c in (config_from_dict(new["config"]), config_from_dict(old["config"])))
        assert abs(a["weight_bytes"] / b["weight_bytes"] - 1.0) < 0.03
        needs = tensor_needs_of_spec(config_from_dict(new["config"]).to_model_spec())
        stored = sum(math.prod(16 if d is None else d for d in n.shape) for k, n in needs.items() if len(n.shape) == 2 and ".conv" not in k and k != "embed")
        assert abs(2 * stored / a["weight_bytes"] - 1.0) < 0.01       # the count of the arithmetic is the count of the tensors
