"""Satavik without a GPU: the configuration reader, the model as data (run order, shared cache entries, tensor names),
the cache's accounting for chunked keys, and the plain implementation against itself and on hand-made inputs."""
import copy
import math

import pytest
import torch

import plain_satavik as P
import satavik_cases as C
from etalii.dllm_b200 import architectures  # noqa: F401
from etalii.dllm_b200.cache.paged import CacheNeed, PagedCache
from etalii.dllm_b200.config.registry import ConfigError, architecture, config_from_dict
from etalii.dllm_b200.weights.loader import expected_tensors


@pytest.mark.parametrize("case", sorted(C.CASES))
def test_config_reads_back_and_names_every_tensor(case):
    config_dict = C.CASES[case]()
    config = config_from_dict(config_dict)
    assert config.model_type == "Satavik" and config.to_hf() == config_dict
    assert config_from_dict(config.to_hf()) == config
    spec = architecture(config.model_type).build_spec(config)
    expected = expected_tensors(spec)
    made = C.random_weights(config_dict)
    assert set(expected) == set(made)
    assert all(tuple(expected[name].shape) == tuple(made[name].shape) for name in made)


def test_a_layer_that_borrows_keys_shares_the_cache_entry_and_writes_nothing():
    config = config_from_dict(C.CASES["borrowed"]())
    spec = architecture("Satavik").build_spec(config)
    order = spec.run_order()
    assert [e.layer for e in order] == [0, 1, 2, 3]
    assert [e.cache for e in order] == [0, 1, 0, 1]
    assert [e.writes_cache for e in order] == [True, True, False, False]
    assert [layer.block for layer in spec.layers] == ["output_norm", "output_norm", "output_norm_mixer", "output_norm"]
    names = expected_tensors(spec)
    assert "l2.mix.k" not in names and "l2.mix.k.norm" not in names and "l2.mix.v" not in names
    assert "l2.mix.q.norm" in names and "l2.norm2" not in names and "l1.mlp.shared.gate" not in names


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="window"), "type 'window' is not supported"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "no keys and values of its own"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top 6 of 5"),
    (lambda c: c.pop("norm"), "no norm"),
])
def test_refused_configurations(change, text):
    config_dict = copy.deepcopy(C.CASES["borrowed"]())
    change(config_dict)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(config_dict)


def test_pages_of_finished_chunks_go_back_to_the_pool():
    """Keys of chunks of 100 positions in pages of 64: a sequence never reads behind the start of the chunk its next
    token lies in, so those pages return while it runs; a whole prompt still gets all its pages at once."""
    need = CacheNeed("kv", kv_heads=1, head_dim=8, value_dim=4, chunk=100)
    cache = PagedCache([need], max_tokens=64 * 12, max_length=64 * 8, max_slots=2)
    slot = cache.acquire(1)[0]
    cache.reserve(slot, 330)  # one step: the tokens of earlier chunks read their own chunks in this step
    cache.advance(slot, 330)
    assert cache.pages_held() == 6
    cache.reserve(slot, 1)  # position 330 lies in the chunk that starts at 300, which is in page 4
    cache.advance(slot, 1)
    assert cache.pages_held() == 2 and cache._groups[0].pages_of[slot][:4] == [None] * 4
    for _ in range(331, 400):
        cache.reserve(slot, 1)
        cache.advance(slot, 1)
    assert cache.pages_held() == 3  # pages 4, 5, 6: position 399 is in page 6
    cache.reserve(slot, 1)  # position 400 starts a chunk in page 6
    assert cache.pages_held() == 1
    cache.check()
    cache.release([slot])
    assert cache.pages_held() == 0
    cache.check()


def test_an_entry_with_several_readers_keeps_what_any_of_them_still_sees():
    """Readers with chunks of 70 and of 100 positions: at position 130 the first still sees from 70 on (page 1), the
    second from 100; at 140 both chunks begin at or after 100 (page 1 still), at 200 the earliest start is 140 (page 2).
    And the design's layers hand their masks to the layer whose cache they read."""
    need = CacheNeed("kv", kv_heads=1, head_dim=8, chunk=(70, 100))
    cache = PagedCache([need], max_tokens=64 * 12, max_length=64 * 8, max_slots=2)
    slot = cache.acquire(1)[0]
    for length, held in ((130, 3), (1, 2), (9, 2), (60, 3), (10, 2)):  # lengths 130, 131, 140, 200, 210
        cache.reserve(slot, length)
        cache.advance(slot, length)
        assert cache.pages_held() == held, (cache.length(slot), cache.pages_held())
    cache.check()
    config = config_from_dict(C.CASES["borrowed"]())
    spec = architecture("Satavik").build_spec(config)
    assert spec.layers[0].parts["mixer"].params["reader_chunks"] == (48, 33)
    assert spec.layers[1].parts["mixer"].params["reader_chunks"] == (70, 1000)


@pytest.mark.parametrize("case", sorted(C.CASES))
def test_plain_model_does_not_depend_on_the_cut(case):
    config_dict = C.CASES[case]()
    weights = C.random_weights(config_dict, 3)
    tokens = C.tokens_for(config_dict, [83])[0]
    whole, layers = P.PlainSatavik(config_dict, weights).feed(tokens, keep_layers=True)
    assert layers.shape[:2] == (len(config_dict["layers"]), 83)
    model, rows = P.PlainSatavik(config_dict, weights), []
    for begin, end in ((0, 1), (1, 3), (3, 48), (48, 49), (49, 83)):
        rows.append(model.feed(tokens[begin:end]))
    assert torch.allclose(torch.cat(rows), whole, rtol=0, atol=1e-9)


def test_plain_mechanisms_on_hand_made_inputs():
    # chunks count from position 0: position 7 with chunks of 4 sees 4..7, position 8 only itself
    assert list(P.visible(7, 4)) == [4, 5, 6, 7] and list(P.visible(8, 4)) == [8] and list(P.visible(2, 4)) == [0, 1, 2]
    # halves: place 0 turns with place 2 (dims 4), place 1 with place 3 at the slower frequency; place 4 stays
    x = torch.tensor([[1.0, 1.0, 0.0, 0.0, 9.0]], dtype=P.F64)
    turned = P.rotate_halves(x, torch.tensor([3]), 4, 100.0)
    assert torch.allclose(turned[0], torch.tensor([math.cos(3.0), math.cos(0.3), math.sin(3.0), math.sin(0.3), 9.0],
                                                  dtype=P.F64))
    # the cap: small scores pass, large ones end at the cap
    assert torch.allclose(P.capped(torch.tensor([0.01, 1000.0], dtype=P.F64), 5.0),
                          torch.tensor([0.01, 5.0], dtype=P.F64), atol=1e-6)
    # the difference weight: equal vectors for both maps leave diff alone
    same = {name: torch.full((4,), 0.5) for name in ("lq1", "lk1", "lq2", "lk2")}
    assert P.difference_weight(same, 0.3) == pytest.approx(0.3)
    same["lk1"] = torch.zeros(4)
    assert P.difference_weight(same, 0.3) == pytest.approx(1.0 - math.e + 0.3)
    # the router: the largest logits, weights a softmax over those only; the bias counts
    w = {"router": torch.eye(4, dtype=P.F64), "router.b": torch.tensor([0.0, 0.0, 0.0, 10.0], dtype=P.F64)}
    chosen, weights = P.route(w, torch.tensor([[3.0, 1.0, 2.0, 0.0]], dtype=P.F64), 2)
    assert chosen.tolist() == [[3, 0]]
    assert torch.allclose(weights, torch.softmax(torch.tensor([[10.0, 3.0]], dtype=P.F64), dim=-1))
    # an expert: the gate is clamped from above only, the up value from both sides
    e = {"e0.gate": torch.eye(2, dtype=P.F64), "e0.up": torch.eye(2, dtype=P.F64), "e0.down": torch.eye(2, dtype=P.F64)}
    out = P.clamped_expert(e, "e0.", torch.tensor([[5.0, -5.0]], dtype=P.F64), 1.0)
    assert torch.allclose(out, torch.tensor([[2.0 / (1 + math.exp(-1.702)), 0.0]], dtype=P.F64), atol=1e-3)
