"""The Dulotar configuration on the CPU: the reader of its keys, what it refuses, and the model it describes."""

import copy

import pytest

from dulotar_tools import CONFIGS, clean
from quantinfer_b200.config import DulotarConfig, config_from_dict
from quantinfer_b200.engine.model import tensor_needs_of_spec
from quantinfer_b200.errors import ConfigError


def test_the_registry_finds_the_class_and_the_dictionary_comes_back():
    for name, cfg in CONFIGS.items():
        c = config_from_dict(clean(cfg))
        assert isinstance(c, DulotarConfig)
        assert c.to_dict() == clean(cfg)
        rebuilt = DulotarConfig(**{k: getattr(c, k) for k in ("vocab", "width", "norm_eps", "embedding_scale", "canon_taps", "layers")})
        assert DulotarConfig.from_dict(rebuilt.to_dict()) == c


def test_the_model_it_describes():
    c = config_from_dict(clean(CONFIGS["U"]))
    s = c.to_model_spec()
    assert len(s.layers) == 3 and [call.layer for call in s.order] == [0, 1, 2, 1, 2]
    assert [call.cache for call in s.order] == [0, 1, 2, 3, 4] and all(call.writes_cache for call in s.order)
    assert s.embedding.scale == 2.5 and s.final_norm.kind == "layernorm" and s.final_norm.eps == 3e-6
    par = s.layers[0]
    assert par.kind == "prenorm_conv" and par.conv.taps == 5 and par.conv.names == ("l0.canon1",) and par.ffn.activation == "relu2"
    l, r = par.mixer.left, par.mixer.right
    assert (l.num_heads, l.num_kv_heads, l.head_dim, l.value_dim, l.chunk, l.conv_taps, l.softcap, l.out_scale) == (6, 3, 10, 6, 9, 2, 4.0, 0.8)
    assert (l.position.rotary_dim, l.position.theta, l.position.pairing, l.bias, l.out_gate) == (4, 300.0, "interleaved", False, False)
    assert (r.heads, r.head_dim, r.value_dim, r.decays, r.out_scale, r.norm_eps) == (3, 5, 7, (0.5, 0.9, 0.97), 1.3, 3e-6)
    assert s.layers[1].mixer.kind == "time_mix" and s.layers[1].ffn is None and s.layers[1].mixer.decay_rank is None
    assert s.layers[2].mixer.kind == "mingru" and s.layers[2].mixer.width == 30
    needs = tensor_needs_of_spec(s)
    assert not any(n.startswith(("l3.", "l4.")) for n in needs)
    assert needs["l1.mix.w1"].shape == (None, 44) and needs["l1.mix.w2"].shape == (18, None) and needs["l1.mix.u"].shape == (3, 6)
    assert needs["l0.mix.left.k.conv"].shape == (30, 2) and needs["l0.mix.right.v"].shape == (21, 44) and needs["l0.norm2.b"].shape == (44,)
    # without the optional keys: no input convolution, no convolution on q, k, v, no cap, no chunks, no rotation
    w = config_from_dict(clean(CONFIGS["W"])).to_model_spec()
    assert w.layers[0].conv is None and w.layers[0].mixer.left.chunk is None and w.layers[0].mixer.left.position is None
    v = config_from_dict(clean(CONFIGS["V"])).to_model_spec()
    assert v.layers[1].mixer.left.conv_taps is None and v.layers[1].mixer.left.softcap is None


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].update(type="attention"), "mixers"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(heads=5), "multiple"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=3), "even"),
    (lambda d: d["layers"][0]["mixer"]["left"]["rot"].update(dims=12), "within"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.9]), "one decay"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.9, 1.5]), "0..1"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(softcap=0.0), "softcap"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(conv=40), "conv"),
    (lambda d: d["layers"][3].update(weights_of=3), "weights_of"),
    (lambda d: d["layers"][3].update(weights_of=4), "weights_of"),
    (lambda d: d["layers"][3].update(weights_of=2), "equal"),
    (lambda d: d["layers"][2].update(mlp={"kind": "moe"}), "dense"),
    (lambda d: d["canon"].update(taps=0), "taps"),
    (lambda d: d["norm"].update(eps=0.0), "eps"),
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["layers"][1]["mixer"].pop("dim"), "dim"),
])
def test_what_it_refuses(edit, word):
    d = copy.deepcopy(clean(CONFIGS["U"]))
    edit(d)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert word in str(e.value)


def test_a_free_dimension_in_a_tensor_need():
    from quantinfer_b200.weights.loader import TensorNeed
    from quantinfer_b200.weights.random_weights import random_tensor

    need = TensorNeed((None, 44))
    assert need.fits((5, 44)) and need.fits((16, 44)) and not need.fits((5, 40)) and not need.fits((44,))
    assert tuple(random_tensor(need, 0, 0, __import__("torch").float32).shape) == (16, 44)


def test_segments_of_long_entries_fill_whole_waves():
    """The length of a segment is chosen on the host from the step's entries: by the count the function's docstring gives,
    a launch of whole waves beats one with a short tail, short entries stay whole, and without a figure for the device
    the fixed length is used."""
    from types import SimpleNamespace

    from quantinfer_b200.parts import segments

    def batch(lens):
        q = [0]
        for n in lens:
            q.append(q[-1] + n)
        return SimpleNamespace(h_q_start=q, extra={}, max_q_len=max(lens))

    assert segments.segment_length(batch([2048]), 32, 0) == segments.SEGMENT
    n = segments.segment_length(batch([2048]), 32, 888)
    assert n % 8 == 0 and 32 <= n <= 256 and -(-2048 // n) * 32 <= 888 < -(-2048 // (n - 8)) * 32      # the shortest that still fits one wave
    # entries below the bound count as one segment each, whatever the length
    b = batch([100, 1, 1, 700])
    n = segments.segment_length(b, 4, 60)
    assert (3 + -(-700 // n)) * 4 <= 60 < (3 + -(-700 // (n - 8))) * 4
    assert segments.segment_length(b, 4, 60) == n and len(b.extra) == 1          # kept for the step's other layers
    # a device that holds everything at once: short segments win until the chain's walk weighs more
    assert segments.segment_length(batch([4096]), 1, 100000) == 32
