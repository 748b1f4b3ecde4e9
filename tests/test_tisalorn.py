"""Tisalorn without a GPU: the configuration reader, the model as data (run order, cache entries, tensor names), and
the plain implementation against itself (a prompt cut anywhere gives what the whole prompt gives)."""
import copy

import pytest
import torch

import plain_tisalorn as P
import tisalorn_cases as C
from etalii.dllm_b200 import architectures  # noqa: F401
from etalii.dllm_b200.config.registry import ConfigError, architecture, config_from_dict
from etalii.dllm_b200.weights.loader import expected_tensors


@pytest.mark.parametrize("case", sorted(C.CASES))
def test_config_reads_back_and_names_every_tensor(case):
    config_dict = C.CASES[case]()
    config = config_from_dict(config_dict)
    assert config.model_type == "Tisalorn" and config.to_hf() == config_dict
    assert config_from_dict(config.to_hf()) == config
    spec = architecture(config.model_type).build_spec(config)
    expected = expected_tensors(spec)
    made = C.random_weights(config_dict)
    assert set(expected) == set(made)
    assert all(tuple(expected[name].shape) == tuple(made[name].shape) for name in made)


def test_run_order_of_a_loop():
    config = config_from_dict(C.config([C.delta(), C.lightning(), C.parallel(), C.delta()], loop=(1, 3, 2)))
    order = architecture("Tisalorn").build_spec(config).run_order()
    assert [e.layer for e in order] == [0, 1, 2, 1, 2, 3]
    assert [e.cache for e in order] == list(range(6))  # every run has a cache entry of its own
    assert [e.reentry for e in order] == [None, 0, None, 0, None, None]
    assert [e.round for e in order] == [0, 0, 0, 1, 1, 0]


def test_no_loop_means_every_layer_once():
    config = config_from_dict(C.config([C.lightning(), C.delta()]))
    spec = architecture("Tisalorn").build_spec(config)
    assert [e.layer for e in spec.run_order()] == [0, 1] and spec.reentries == ()


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="window"), "type 'window' is not supported"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(vdim=16), "values are the keys"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "one decay per head"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "mlp.kind"),
    (lambda c: c.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda c: c.pop("norm"), "no norm"),
])
def test_refused_configurations(change, text):
    config_dict = copy.deepcopy(C.CASES["mixed"]())
    change(config_dict)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(config_dict)


@pytest.mark.parametrize("case", sorted(C.CASES))
def test_plain_model_does_not_depend_on_the_cut(case):
    config_dict = C.CASES[case]()
    model = P.PlainTisalorn(config_dict, C.random_weights(config_dict, 3))
    tokens = C.tokens_for(config_dict, [23])[0]
    whole, layers = model.forward(tokens, {})
    assert layers.shape[0] == len(model.before) + sum(len(i) for _, i in model.passes) + len(model.after)
    cache, rows = {}, []
    for begin, end in ((0, 1), (1, 3), (3, 11), (11, 12), (12, 23)):
        rows.append(model.forward(tokens[begin:end], cache)[0])
    assert torch.allclose(torch.cat(rows), whole, rtol=0, atol=1e-9)


def test_plain_mechanisms_on_hand_made_inputs():
    # a decay of zero keeps only the current token: o_t = (k_t . q_t) v_t
    q, k, v = torch.randn(5, 1, 4, dtype=P.F64), torch.randn(5, 1, 4, dtype=P.F64), torch.randn(5, 1, 3, dtype=P.F64)
    out = P.decayed_outer_product_scan(q, k, v, torch.zeros(1, dtype=P.F64), torch.zeros(1, 4, 3, dtype=P.F64))
    assert torch.allclose(out[:, 0], (q * k).sum(-1) * v[:, 0])
    # the convolution's last tap multiplies the token itself, and zeros stand before the start
    y, history = P.short_convolution(torch.tensor([[1.0], [2.0], [3.0]], dtype=P.F64),
                                     torch.tensor([[100.0, 10.0, 1.0]], dtype=P.F64), torch.zeros(2, 1, dtype=P.F64))
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0] and history[:, 0].tolist() == [2.0, 3.0]
    # interleaved pairs: dimension 0 turns with dimension 1 by the position's angle (frequency 1 for pair 0)
    x = torch.tensor([[[1.0, 0.0, 5.0, 7.0]]], dtype=P.F64)
    turned = P.rotate_interleaved(x, torch.tensor([2]), 2, 10000.0)
    assert torch.allclose(turned[0, 0], torch.tensor([torch.cos(torch.tensor(2.0)), torch.sin(torch.tensor(2.0)), 5.0,
                                                      7.0], dtype=P.F64))
    # the clamp: gate only from above, up from both sides
    w = {"gate": torch.eye(2, dtype=P.F64), "up": torch.eye(2, dtype=P.F64), "down": torch.eye(2, dtype=P.F64)}
    out = P.clamped_glu(w, {"limit": 1.0}, torch.tensor([[5.0, -5.0]], dtype=P.F64))
    assert torch.allclose(out, torch.tensor([[1.0 / (1 + torch.exp(torch.tensor(-1.702))) * 2.0, 0.0]], dtype=P.F64),
                          atol=1e-3)
