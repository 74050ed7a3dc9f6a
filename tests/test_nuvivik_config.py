"""The Nuvivik configuration reader, the checkpoint's tensor list, the stretched rotation
frequencies, and what the windowed mixers ask of the cache manager (no GPU)."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_nuvivik as pn
from forge_engine_b200.config import read_model_config
from forge_engine_b200.errors import ConfigError


def example():
    return pn.config([
        pn.latent_layer(window=11),
        pn.attention_layer(window=7, scaling=(4.0, 1.0, 3.0, 24), mlp=pn.routed()),
        pn.latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=24, kv_rank=16, window=19, mlp=None),
        pn.attention_layer(heads=6, kv_heads=2, dim=8, vdim=12, window=13, rot_dims=8, softcap=None, mlp=pn.routed(groups=None, top=1)),
    ])


def test_registry_finds_the_architecture_and_reads_every_constant():
    arch, cfg, spec = read_model_config(example())
    assert arch.name == "Nuvivik" and spec.vocab_size == 97 and spec.hidden_size == 64
    assert spec.embedding_scale == 0.7 and spec.logit_scale == 1.5 and spec.logit_softcap == 25.0
    assert not spec.tie_embeddings and spec.position_table_name is None
    first, second, third, fourth = spec.layers
    assert all(layer.arrangement == "output_norm" and layer.input_norm is None and layer.post_norm is None for layer in spec.layers)
    assert first.options.mixer_out_norm.eps == 1e-5 and first.options.mixer_out_norm.weight_offset == 0.0
    latent = first.mixer
    assert latent.kind == "latent_attention" and latent.window == 11 and latent.sink
    assert (latent.num_heads, latent.head_dim, latent.rot_dim, latent.v_head_dim, latent.q_rank, latent.kv_rank) == (3, 16, 8, 24, 32, 40)
    assert latent.position.rotary_dim == 8 and not latent.position.interleaved and latent.position.scaling is None
    assert first.ffn.kind == "dense_mlp" and first.ffn.activation == "gelu_tanh" and not first.ffn.bias and first.ffn.intermediate_size == 48
    attention = second.mixer
    assert (attention.num_heads, attention.num_kv_heads, attention.head_dim, attention.v_head_dim) == (4, 2, 16, 16)
    assert attention.bias and attention.o_bias is False and attention.window == 7 and attention.softcap == 15.0
    assert attention.qk_norm and not attention.qk_norm_weight and attention.qk_norm_after_rotation
    assert attention.position.rotary_dim == 8 and attention.position.scaling == (4.0, 1.0, 3.0, 24.0) and attention.position.theta == 10000.0
    routed = second.ffn
    assert (routed.experts, routed.top, routed.groups, routed.group_score) == (6, 2, (3, 2), "top2")
    assert routed.score == "sigmoid" and not routed.renormalise and routed.weight_on == "output" and routed.shared is None
    assert routed.expert.kind == "dense_mlp" and routed.expert.activation == "relu2" and routed.expert.intermediate_size == 24
    assert third.ffn is None and third.options.ffn_out_norm is None and third.mixer.window == 19
    assert fourth.mixer.softcap is None and fourth.mixer.position.scaling is None and fourth.ffn.groups is None and fourth.ffn.top == 1
    assert [run.layer for run in spec.schedule] == [0, 1, 2, 3] and all(run.cache_of is None for run in spec.schedule)


def test_constants_that_may_be_left_out():
    raw = example()
    del raw["logit_softcap"], raw["logit_scale"], raw["embedding"]
    _, _, spec = read_model_config(raw)
    assert spec.logit_softcap is None and spec.logit_scale == 1.0 and spec.embedding_scale == 1.0


def test_expected_tensors_are_the_checkpoints():
    full = example()
    arch, _, spec = read_model_config(full)
    expected = arch.expected_tensors(spec)
    shapes = pn.tensor_shapes(full)
    assert set(expected) == set(shapes)
    for name, shape in shapes.items():
        assert tuple(expected[name].shape) == tuple(shape), name
    assert "l1.mix.o.b" not in expected and "l1.mix.q.b" in expected and "l0.mix.sink" in expected
    assert "l2.norm2" not in expected and "l1.mlp.e0.gate" not in expected


@pytest.mark.parametrize("path, value", (
    (("layers", 0, "type"), "attention2"),
    (("layers", 1, "mixer", "kv_heads"), 3),
    (("layers", 1, "mixer", "rot", "dims"), 7),
    (("layers", 1, "mixer", "rot", "dims"), 18),
    (("layers", 1, "mixer", "rot", "scaling", "high"), 1.0),
    (("layers", 1, "mixer", "rot", "scaling", "factor"), 0.0),
    (("layers", 1, "mixer", "softcap"), 0.0),
    (("layers", 1, "mixer", "mask", "size"), 0),
    (("layers", 0, "mixer", "rot", "dims"), 4),
    (("layers", 0, "mixer", "kv_rank"), 0),
    (("layers", 1, "mlp", "router", "top"), 5),
    (("layers", 1, "mlp", "router", "groups", "count"), 4),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4),
    (("layers", 1, "mlp", "kind"), "sparse"),
    (("norm", "eps"), 0.0),
    (("logit_softcap",), -1.0),
))
def test_bad_values_are_refused(path, value):
    raw = copy.deepcopy(example())
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError):
        read_model_config(raw)


@pytest.mark.parametrize("dims, base, scaling", ((16, 50000.0, (8.0, 1.0, 4.0, 1024)), (32, 10000.0, (4.0, 2.0, 5.0, 200)),
                                                  (8, 100.0, (2.0, 1.0, 1.5, 16)), (64, 500000.0, (32.0, 1.0, 4.0, 8192)), (6, 10.0, None)))
def test_stretched_frequencies(dims, base, scaling):
    """The rotation's frequencies with every branch of the stretch: kept, divided, blended."""
    from forge_engine_b200.config.specs import RotarySpec
    from forge_engine_b200.parts.base import BuildContext, build_part

    ctx = BuildContext(dtype=torch.float32, device=torch.device("cpu"), status=None)
    rot = {"dims": dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    want = torch.tensor(pn.frequencies(rot), dtype=torch.float64)
    part = build_part(RotarySpec(dims, base, dims, scaling=scaling, exact_frequencies=True), {}, ctx)
    got = part.rotary()[0].double()
    assert part.rotary()[1] == dims and float(((got - want) / want).abs().max()) < 1e-6
    if scaling is not None:
        plain = torch.tensor(pn.frequencies({"dims": dims, "base": base}), dtype=torch.float64)
        changed = want != plain
        blended = changed & ((want - plain / scaling[0]).abs() > 1e-12 * plain)
        assert bool(changed.any()) and bool((~changed).any()), "both a kept and a stretched frequency occur"
        assert bool(blended.any()) or dims < 16, "a blended frequency occurs"


def test_windowed_mixers_give_their_pages_back():
    """Both mixers tell the cache manager their window: a request's pages before it are
    released, and a layer group exists per distinct (heads, size, window)."""
    from forge_engine_b200.cache.manager import CacheManager, PagedKVSpec

    _, _, spec = read_model_config(example())
    from forge_engine_b200.parts.attention import GQAttention
    from forge_engine_b200.parts.latent_attention import LatentAttention

    kinds = {"gqa_attention": GQAttention, "latent_attention": LatentAttention}
    needs = []
    for layer in spec.layers:
        mixer = object.__new__(kinds[layer.mixer.kind])
        m = layer.mixer
        if m.kind == "latent_attention":
            mixer.kv_rank, mixer.r, mixer.window = m.kv_rank, m.rot_dim, m.window
        else:
            mixer.spec, mixer.nkv, mixer.d, mixer.dv, mixer.parts, mixer.keep_first = m, m.num_kv_heads, m.head_dim, m.v_head_dim, 1, 0
        needs.append(mixer.cache_needs())
    assert [n.kv.window for n in needs] == [11, 7, 19, 13]
    assert needs[0].kv == PagedKVSpec(1, 48, 11, 0) and needs[3].kv == PagedKVSpec(2, 8, 13, 12, 0)
    cache = CacheManager(needs, page_size=4, num_pages=40, max_requests=2, device="cpu", dtype=torch.float32)
    cache.begin_request("a")
    cache.reserve("a", 40)
    cache.advance("a", 40)
    held = cache.request("a")
    live = [sum(1 for p in table.pages if p >= 0) for table in held.tables]
    assert all(n < 10 for n in live) and len(set(live)) > 1       # 10 pages hold 40 tokens; every window keeps fewer
    cache.check_consistency()
    cache.end_request("a")
    assert all(n == 0 for n in cache.leased_pages())
