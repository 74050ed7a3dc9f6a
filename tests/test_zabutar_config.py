"""The Zabutar configuration reader, the checkpoint's tensor list, the table of biases by
distance, and the cache manager's state that stays a run's own where it reads another run's
keys and values (no GPU)."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_zabutar as pz
from forge_engine_b200.cache.manager import CacheManager, CacheNeeds, PagedKVSpec, StateSpec
from forge_engine_b200.config import read_model_config
from forge_engine_b200.errors import ConfigError


def example():
    return pz.written(pz.config([
        pz.recurrent_layer(), pz.attention_layer(mlp=pz.routed()), pz.recurrent_layer(mlp=None),
        pz.attention_layer(kv_from=1, bias_max=17.5, mlp=pz.routed(identity=0, experts=6, shared_ff=None))], taps=4))


def test_registry_finds_the_architecture_and_reads_every_constant():
    arch, cfg, spec = read_model_config(example())
    assert arch.name == "Zabutar" and spec.vocab_size == 97 and spec.hidden_size == 64 and spec.max_positions == 512
    assert spec.position_table_name == "pos" and not spec.tie_embeddings
    first, second, third, fourth = spec.layers
    assert all(layer.arrangement == "sandwich_conv" and layer.options.taps == 4 for layer in spec.layers)
    assert first.input_norm.weight_offset == 1.0 and first.options.mixer_out_norm.weight_offset == 1.0
    assert first.mixer.kind == "gated_recurrence"
    assert (first.mixer.num_heads, first.mixer.head_dim, first.mixer.v_head_dim) == (4, 8, 16)
    assert first.ffn.kind == "dense_mlp" and first.ffn.intermediate_size == 48 and first.ffn.bias
    attention = second.mixer
    assert (attention.num_heads, attention.num_kv_heads, attention.head_dim, attention.v_head_dim) == (4, 2, 16, 16)
    assert attention.scale == 0.25 and attention.distance_bias_table == (None, 40.0) and attention.kv_projection
    assert attention.position.kind == "none" and attention.window is None
    routed = second.ffn
    assert (routed.experts, routed.identity, routed.top, routed.groups) == (5, 1, 2, (3, 2))
    assert routed.score == "softmax" and routed.renormalise and routed.weight_on == "output" and routed.correction
    assert routed.weight_scale == 1.5 and routed.renorm_floor == 1e-20 and routed.shared.intermediate_size == 40
    assert third.ffn is None and third.post_norm is None and third.options.ffn_out_norm is None
    assert not fourth.mixer.kv_projection and fourth.mixer.distance_bias_table == (None, 17.5)
    assert fourth.ffn.identity == 0 and fourth.ffn.shared is None
    assert [run.layer for run in spec.schedule] == [0, 1, 2, 3]
    assert [run.cache_of for run in spec.schedule] == [None, None, None, 1]


def test_expected_tensors_are_the_checkpoints():
    full = pz.config([pz.recurrent_layer(), pz.attention_layer(mlp=pz.routed()), pz.recurrent_layer(mlp=None),
                      pz.attention_layer(kv_from=1, mlp=pz.routed(identity=0, experts=6, shared_ff=None))])
    arch, _, spec = read_model_config(pz.written(full))
    expected = arch.expected_tensors(spec)
    shapes = pz.tensor_shapes(full)
    assert set(expected) == set(shapes)
    for name, shape in shapes.items():
        wanted = tuple(expected[name].shape)
        # the rows of the bias table are the stored tensor's: the model leaves them open
        assert len(wanted) == len(shape) and all(w is None or w == s for w, s in zip(wanted, shape)), name
    assert tuple(expected["l1.mix.rel"].shape) == (None, 4)
    assert "l3.mix.k" not in expected and "l3.mix.v" not in expected and "l3.mix.rel" in expected


@pytest.mark.parametrize("path, value", (
    (("layers", 0, "type"), "hgrn3"),
    (("layers", 1, "mixer", "kv_heads"), 3),
    (("layers", 1, "mixer", "bias_max"), 1.0),
    (("layers", 3, "mixer", "kv_from"), 0),
    (("layers", 3, "mixer", "kv_from"), 3),
    (("layers", 3, "mixer", "kv_heads"), 4),
    (("layers", 3, "mixer", "dim"), 32),
    (("layers", 1, "mlp", "router", "top"), 5),
    (("layers", 1, "mlp", "router", "groups", "count"), 4),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4),
    (("layers", 1, "mlp", "kind"), "sparse"),
    (("canon", "taps"), 0),
    (("norm", "eps"), 0.0),
))
def test_bad_values_are_refused(path, value):
    raw = copy.deepcopy(example())
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        read_model_config(raw)


@pytest.mark.parametrize("rows, far", ((12, 40), (30, 140), (8, 17.5), (2, 9), (4, 3), (6, 250), (64, 1000.5), (10, 5.01)))
def test_distance_bias_is_expanded_bucket_by_bucket(rows, far):
    from forge_engine_b200.parts.attention import GQAttention

    stored = torch.randn(rows, 3, generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16)
    table = GQAttention.expand_distance_bias(stored, far)
    assert table.dtype == torch.float32 and table.shape[0] == 3
    reach = table.shape[1]
    assert pz.distance_bucket(reach - 1, rows, far) == rows - 1 and (reach < 2 or pz.distance_bucket(reach - 2, rows, far) < rows - 1)
    for n in range(int(far) + 50):
        want = stored.float()[pz.distance_bucket(n, rows, far)]
        assert torch.equal(table[:, min(n, reach - 1)], want), n


def test_a_run_that_reads_another_runs_pages_keeps_a_state_of_its_own():
    kv = PagedKVSpec(2, 16, None)
    conv = StateSpec((2, 3, 8), "float32")
    needs = [CacheNeeds(kv=kv, own_state=conv), CacheNeeds(state=StateSpec((2, 4, 4)), own_state=conv),
             CacheNeeds(kv=kv, own_state=conv), CacheNeeds()]
    cache = CacheManager(needs, page_size=4, num_pages=8, max_requests=2, shares={2: 0}, device="cpu", dtype=torch.float32)
    views = [cache.view(run) for run in range(4)]
    assert views[2].group == views[0].group and not views[2].owns and views[0].owns
    assert views[0].own_state.shape == (3, 2, 3, 8) and views[3].own_state is None and views[3].state is None
    pointers = {views[run].own_state.data_ptr() for run in range(3)}
    assert len(pointers) == 3                                  # one per run, the sharing run's too
    assert views[1].state.shape == (3, 2, 4, 4) and views[1].state.data_ptr() not in pointers
    # a slot that is leased again reads as new
    cache.begin_request("a")
    slot = cache.request("a").slot
    for run in range(3):
        cache.view(run).own_state[slot].fill_(5.0)
    cache.end_request("a")
    cache.begin_request("b")
    assert cache.request("b").slot == slot
    assert all(float(cache.view(run).own_state[slot].abs().max()) == 0.0 for run in range(3))
