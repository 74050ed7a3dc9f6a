"""The Nuvivik design in the engine against the plain implementation of ``plain_nuvivik.py``:
every mechanism alone, whole prompts against portions and token-by-token decoding, unequal
batches, reused pages and slots, keys just inside and just outside a window (at page borders,
in prompts and when decoding), tokens far back that reach a late logit through stacked
windows, sinks, the first tokens of a sequence, other sizes, generation."""

from __future__ import annotations

import json
import math

import pytest
import torch
from safetensors.torch import save_file

import plain_nuvivik as pn

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


# -- helpers --------------------------------------------------------------------------------
def write_model(folder, cfg: dict, seed: int, change=None) -> dict:
    weights = pn.random_weights(cfg, seed)
    if change is not None:
        change(weights)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return weights


def make_runner(folder, dtype: str, page_size=4, num_pages=96, max_requests=4, use_graphs=True):
    from forge_engine_b200.engine import ModelRunner

    return ModelRunner.from_folder(folder, dtype=dtype, page_size=page_size, num_pages=num_pages,
                                   max_requests=max_requests, use_graphs=use_graphs)


def tokens_of(cfg: dict, length: int, seed: int, avoid=()) -> list:
    gen = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, cfg["vocab"] - len(avoid), (length,), generator=gen).tolist()
    spare = [t for t in range(cfg["vocab"]) if t not in avoid]
    return [spare[t] for t in ids]


def run_schedule(runner, requests: dict, schedule: list) -> dict:
    """``schedule``: steps, each a list of (request, number of its next tokens); a request
    begins at its first entry and ends with its last token.  Logits of every position."""
    from forge_engine_b200.engine import StepEntry

    at = {key: 0 for key in requests}
    rows = {key: [] for key in requests}
    for step in schedule:
        entries = []
        for key, count in step:
            if at[key] == 0:
                runner.begin(key)
            entries.append(StepEntry(key, requests[key][at[key] : at[key] + count], list(range(count))))
        logits = runner.step(entries).float().cpu()
        runner.check_status()
        begin = 0
        for key, count in step:
            rows[key].append(logits[begin : begin + count])
            begin += count
            at[key] += count
            if at[key] == len(requests[key]):
                runner.end(key)
        runner.cache.check_consistency()
    assert all(at[key] == len(requests[key]) for key in requests)
    return {key: torch.cat(parts) for key, parts in rows.items()}


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    want = want.float()
    assert got.shape == want.shape, what
    assert torch.isfinite(got).all(), what
    scale = float(want.abs().max())
    if dtype == "float32":
        worst = float((got - want).abs().max())
        assert worst <= 2e-4 * max(1.0, scale), f"{what}: {worst} against a scale of {scale}"
    else:
        error = float(((got - want) ** 2).mean().sqrt() / (want**2).mean().sqrt())
        assert error <= 3e-2, f"{what}: relative error {error}"


def oracle(cfg, weights, tokens) -> torch.Tensor:
    return pn.forward(cfg, weights, tokens)


def all_chosen():
    """A routed feed-forward in which every expert of the kept groups is chosen, so that
    nothing rests on a close call of the router (which bfloat16 rounding decides otherwise)."""
    return pn.routed(experts=3, top=3, ff=32, groups=(1, 1))


def routed_for(dtype: str, **kwargs):
    return pn.routed(**kwargs) if dtype == "float32" else all_chosen()


def mixed_config(dtype: str = "float32"):
    """All mechanisms in one model, the layers' windows, head counts and sizes all different.
    Routers that choose are compared in 32-bit (a close call decided the other way by bfloat16
    rounding changes a token's logits far beyond rounding) and, in bfloat16, on the part alone
    where the margins are known."""
    return pn.config([
        pn.latent_layer(window=11),
        pn.attention_layer(window=7, scaling=(4.0, 1.0, 3.0, 24), mlp=routed_for(dtype)),
        pn.latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=24, kv_rank=16, window=19,
                        mlp=routed_for(dtype, experts=8, top=3, groups=(4, 2))),
        pn.attention_layer(heads=6, kv_heads=2, dim=8, vdim=12, window=13, rot_dims=8, softcap=None, mlp=None),
        pn.latent_layer(window=5, mlp=None),
    ])


# -- every mechanism alone --------------------------------------------------------------------
SINGLE = {
    "attention_dense": [pn.attention_layer()],
    "attention_no_ff": [pn.attention_layer(mlp=None)],
    "attention_no_cap": [pn.attention_layer(softcap=None)],
    "attention_whole_head_rotated": [pn.attention_layer(rot_dims=16)],
    "attention_two_rotated": [pn.attention_layer(rot_dims=2)],
    "attention_stretched": [pn.attention_layer(scaling=(8.0, 1.0, 4.0, 16), base=50.0)],
    "attention_odd_sizes": [pn.attention_layer(heads=3, kv_heads=1, dim=12, vdim=20, rot_dims=6)],
    "attention_heads_of_64": [pn.attention_layer(heads=2, kv_heads=2, dim=64, vdim=64, rot_dims=32)],
    "attention_heads_of_128": [pn.attention_layer(heads=4, kv_heads=1, dim=128, vdim=128, rot_dims=64, softcap=8.0)],
    "attention_wide_values": [pn.attention_layer(heads=2, kv_heads=1, dim=16, vdim=48)],
    "attention_window_of_one": [pn.attention_layer(window=1)],
    "latent_dense": [pn.latent_layer()],
    "latent_no_ff": [pn.latent_layer(mlp=None)],
    "latent_odd_sizes": [pn.latent_layer(heads=3, dim=10, rot_dim=6, vdim=14, q_rank=20, kv_rank=26)],
    "latent_one_head": [pn.latent_layer(heads=1, dim=32, rot_dim=16, vdim=32, q_rank=48, kv_rank=48)],
    "latent_sixteens": [pn.latent_layer(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=32, kv_rank=48)],
    "latent_window_of_two": [pn.latent_layer(window=2)],
    "routed": [pn.latent_layer(mlp=pn.routed())],
    "routed_top_one": [pn.attention_layer(mlp=pn.routed(top=1))],
    "routed_no_groups": [pn.attention_layer(mlp=pn.routed(experts=5, top=2, groups=None))],
    "routed_groups_of_one": [pn.latent_layer(mlp=pn.routed(experts=4, top=2, groups=(4, 3)))],
    "routed_one_group_kept": [pn.latent_layer(mlp=pn.routed(experts=12, top=2, ff=16, groups=(2, 1)))],
    "routed_odd_width_of_experts": [pn.attention_layer(mlp=pn.routed(experts=6, top=2, ff=20, groups=(3, 1)))],
    "routed_all": [pn.latent_layer(mlp=all_chosen())],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    if dtype == "bfloat16" and name.startswith("routed") and name != "routed_all":
        pytest.skip("routers that choose are compared in 32-bit and on the part alone")
    cfg = pn.config(SINGLE[name])
    weights = write_model(tmp_path / "m", cfg, 11)
    tokens = tokens_of(cfg, 37, 5)
    runner = make_runner(tmp_path / "m", dtype)
    got = run_schedule(runner, {"a": tokens}, [[("a", len(tokens))]])["a"]
    assert_close(got, oracle(cfg, weights, tokens), dtype, name)


def test_residual_after_every_layer(tmp_path):
    """The residual stream after every layer, in 32-bit, against the plain implementation."""
    from forge_engine_b200.engine import StepEntry

    cfg = mixed_config()
    weights = write_model(tmp_path / "m", cfg, 12)
    tokens = tokens_of(cfg, 33, 6)
    want = []
    pn.forward(cfg, weights, tokens, layers_out=want)
    runner = make_runner(tmp_path / "m", "float32", use_graphs=False)
    seen = []
    for block in runner.model.blocks:
        inner = block.forward

        def spy(h, pending, batch, cache, inner=inner):
            out = inner(h, pending, batch, cache)
            update, norm = out
            u = update.float()
            seen.append((h + u / torch.sqrt((u * u).mean(-1, keepdim=True) + norm.eps) * norm.weight).cpu())
            return out

        block.forward = spy
    runner.begin("a")
    runner.step([StepEntry("a", tokens, [len(tokens) - 1])])
    runner.check_status()
    assert len(seen) == len(want)
    for index, (got, ref) in enumerate(zip(seen, want)):
        assert float((got - ref.float()).abs().max()) <= 2e-4 * max(1.0, float(ref.abs().max())), f"layer {index}"


def test_constants_outside_the_layers(tmp_path):
    """Embedding scale, logit scale and the logits' cap, each alone and none of them."""
    layers = [pn.attention_layer(), pn.latent_layer()]
    for options in (dict(embedding_scale=1.0, logit_scale=1.0, logit_softcap=None), dict(embedding_scale=3.0, logit_scale=1.0, logit_softcap=None),
                    dict(embedding_scale=1.0, logit_scale=0.25, logit_softcap=None), dict(embedding_scale=1.0, logit_scale=4.0, logit_softcap=2.5)):
        cfg = pn.config(layers, **options)
        weights = write_model(tmp_path / "m", cfg, 31)
        tokens = tokens_of(cfg, 20, 3)
        got = run_schedule(make_runner(tmp_path / "m", "float32"), {"a": tokens}, [[("a", 20)]])["a"]
        assert_close(got, oracle(cfg, weights, tokens), "float32", str(options))
        if options["logit_softcap"] is not None:
            assert float(got.abs().max()) <= options["logit_softcap"] and float(got.abs().max()) > 0.9 * options["logit_softcap"]


# -- the same sequence cut in different ways ------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_against_token_by_token_decoding(tmp_path, dtype):
    cfg = mixed_config(dtype)
    weights = write_model(tmp_path / "m", cfg, 13)
    tokens = tokens_of(cfg, 45, 7)
    runner = make_runner(tmp_path / "m", dtype)
    ref = oracle(cfg, weights, tokens)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 45)]])["a"]
    single = run_schedule(runner, {"b": tokens}, [[("b", 1)] for _ in range(45)])["b"]
    assert_close(whole, ref, dtype, "whole prompt")
    assert_close(single, ref, dtype, "token by token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", ((7, 2, 13, 3, 2, 5, 1, 16, 2, 9), (2,) * 20, (1, 2, 1, 3, 30, 2), (33, 2, 2, 2)))
def test_portions_of_several_sizes(tmp_path, sizes, dtype):
    """Portions down to two tokens (and one), cut in the middle of pages and windows."""
    cfg = mixed_config(dtype)
    weights = write_model(tmp_path / "m", cfg, 14)
    tokens = tokens_of(cfg, sum(sizes), 8)
    runner = make_runner(tmp_path / "m", dtype)
    got = run_schedule(runner, {"a": tokens}, [[("a", n)] for n in sizes])["a"]
    assert_close(got, oracle(cfg, weights, tokens), dtype, f"portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_against_each_alone(tmp_path, dtype):
    cfg = mixed_config(dtype)
    weights = write_model(tmp_path / "m", cfg, 15)
    requests = {"a": tokens_of(cfg, 41, 1), "b": tokens_of(cfg, 9, 2), "c": tokens_of(cfg, 23, 3), "d": tokens_of(cfg, 3, 4)}
    schedule = [
        [("a", 17), ("b", 2)],
        [("a", 1), ("b", 1), ("c", 20)],
        [("c", 2), ("a", 20), ("d", 2), ("b", 5)],
        [("d", 1), ("a", 3), ("b", 1), ("c", 1)],
    ]
    runner = make_runner(tmp_path / "m", dtype)
    together = run_schedule(runner, requests, schedule)
    for key, tokens in requests.items():
        alone = run_schedule(runner, {key: tokens}, [[(key, len(tokens))]])[key]
        assert_close(together[key], oracle(cfg, weights, tokens), dtype, f"request {key} in the batch")
        if dtype == "float32":
            assert float((together[key] - alone).abs().max()) <= 1e-4 * max(1.0, float(alone.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_slots_freed_and_used_again(tmp_path, dtype):
    """Two slots and a small pool: later requests get the pages of earlier ones (and pages that
    a window has given back in the middle of a request), which must read as new."""
    cfg = mixed_config(dtype)
    weights = write_model(tmp_path / "m", cfg, 16)
    requests = {key: tokens_of(cfg, n, i) for i, (key, n) in enumerate((("a", 22), ("b", 31), ("c", 27), ("d", 9)))}
    schedule = [
        [("a", 20), ("b", 3)],
        [("a", 2), ("b", 20)],          # a ends
        [("c", 11), ("b", 1)],          # c takes a's slot and pages
        [("b", 7), ("c", 16)],          # both end
        [("d", 9)],
    ]
    runner = make_runner(tmp_path / "m", dtype, page_size=4, num_pages=16, max_requests=2)
    got = run_schedule(runner, requests, schedule)
    assert runner.cache.slots.leased_count == 0 and all(n == 0 for n in runner.cache.leased_pages())
    for key, tokens in requests.items():
        assert_close(got[key], oracle(cfg, weights, tokens), dtype, f"request {key}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path, dtype):
    """A short prompt, then far more single tokens than any window or page holds: every
    window passes over decoded tokens, its pages go back to the pool, and the decode steps
    are replayed from captured graphs."""
    cfg = mixed_config(dtype)
    weights = write_model(tmp_path / "m", cfg, 17)
    tokens = tokens_of(cfg, 120, 9)
    runner = make_runner(tmp_path / "m", dtype, page_size=4, num_pages=40)
    got = run_schedule(runner, {"a": tokens}, [[("a", 5)]] + [[("a", 1)] for _ in range(115)])["a"]
    assert_close(got, oracle(cfg, weights, tokens), dtype, "long decoding")
    if runner.use_graphs:
        assert runner.graphs.captured


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_steps_replayed_from_graphs(tmp_path, dtype):
    """Steps that bring a prompt portion beside two decoding requests, captured at first sight
    and replayed (filler entries pad them to their bucket).  Logits at every entry's last token
    against the plain implementation."""
    from forge_engine_b200.engine import StepEntry

    cfg = mixed_config(dtype)
    weights = write_model(tmp_path / "m", cfg, 18)
    requests = {"a": tokens_of(cfg, 16 * 9 + 5, 1), "b": tokens_of(cfg, 19, 2), "c": tokens_of(cfg, 24, 3)}
    schedule = [[("b", 9), ("c", 14)]] + [[("a", 16), ("b", 1), ("c", 1)] for _ in range(9)] + [[("a", 5), ("b", 1), ("c", 1)]]
    runner = make_runner(tmp_path / "m", dtype, page_size=16, num_pages=40)
    runner.graphs.capture_after = 1
    refs = {key: oracle(cfg, weights, tokens).float() for key, tokens in requests.items()}
    at = {key: 0 for key in requests}
    for step in schedule:
        entries = []
        for key, count in step:
            if at[key] == 0:
                runner.begin(key)
            entries.append(StepEntry(key, requests[key][at[key] : at[key] + count], [count - 1]))
        logits = runner.step(entries).float().cpu()
        runner.check_status()
        for row, (key, count) in enumerate(step):
            at[key] += count
            assert_close(logits[row : row + 1], refs[key][at[key] - 1 : at[key]], dtype, f"{key} at {at[key] - 1}")
    assert len(runner.graphs.captured) >= 1


# -- other sizes ------------------------------------------------------------------------------
OTHER = {
    "narrow": dict(layers=[pn.latent_layer(heads=1, dim=4, rot_dim=2, vdim=4, q_rank=6, kv_rank=6),
                           pn.attention_layer(heads=1, kv_heads=1, dim=8, vdim=8, rot_dims=2)], width=20, vocab=11),
    "width_not_in_eights": dict(layers=[pn.latent_layer(heads=2, dim=6, rot_dim=2, vdim=10, q_rank=12, kv_rank=10),
                                        pn.attention_layer(mlp=pn.routed())], width=36),
    "every_head_its_own_keys": dict(layers=[pn.attention_layer(heads=4, kv_heads=4)]),
    "one_key_head": dict(layers=[pn.attention_layer(heads=8, kv_heads=1, dim=32, vdim=32, rot_dims=8)]),
    "many_heads_per_key_head": dict(layers=[pn.attention_layer(heads=12, kv_heads=1, dim=8, vdim=8, rot_dims=4)]),
    "ranks_differ": dict(layers=[pn.latent_layer(heads=2, dim=16, rot_dim=16, vdim=8, q_rank=16, kv_rank=64)]),
    "wide_latent": dict(layers=[pn.latent_layer(heads=2, dim=24, rot_dim=8, vdim=40, q_rank=96, kv_rank=136)], width=96),
    "scale_one_eps_large": dict(layers=[pn.attention_layer(scale=1.0), pn.latent_layer(scale=1.0)], eps=0.5),
    "windows_longer_than_the_sequence": dict(layers=[pn.attention_layer(window=500), pn.latent_layer(window=64)]),
    "no_mask": dict(layers=[pn.attention_layer(window=None), pn.latent_layer(window=None), pn.attention_layer(heads=2, kv_heads=2, dim=64, vdim=64,
                                                                                                            rot_dims=16, window=None)]),
    "top_equals_experts": dict(layers=[pn.latent_layer(mlp=pn.routed(experts=4, top=4, groups=(2, 2)))]),
    "many_experts": dict(layers=[pn.attention_layer(mlp=pn.routed(experts=40, top=5, ff=8, groups=(8, 3)))]),
    "latent_layers_only": dict(layers=[pn.latent_layer(window=9), pn.latent_layer(window=9, mlp=pn.routed(top=1)), pn.latent_layer(window=9)]),
    "attention_layers_only": dict(layers=[pn.attention_layer(window=3), pn.attention_layer(window=30, mlp=None)]),
}


@pytest.mark.parametrize("name", sorted(OTHER))
def test_other_sizes_and_values_that_are_one_or_equal(tmp_path, name):
    options = dict(OTHER[name])
    cfg = pn.config(options.pop("layers"), **options)
    weights = write_model(tmp_path / "m", cfg, 21)
    tokens = tokens_of(cfg, 50, 10)
    runner = make_runner(tmp_path / "m", "float32", page_size=8, num_pages=24)
    ref = oracle(cfg, weights, tokens)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 50)]])["a"]
    cut = run_schedule(runner, {"b": tokens}, [[("b", 19)], [("b", 2)], [("b", 13)]] + [[("b", 1)] for _ in range(16)])["b"]
    assert_close(whole, ref, "float32", name)
    assert_close(cut, ref, "float32", name + ", cut")


@pytest.mark.parametrize("dtype", DTYPES)
def test_bfloat16_sizes_of_the_tensor_core_paths(tmp_path, dtype):
    """Sizes in sixteens, so that the bfloat16 engine takes its tensor-core products and the
    tensor-core attention kernel, with steps long enough for several row tiles and windows that
    end inside a key tile."""
    cfg = pn.config([pn.latent_layer(heads=4, dim=32, rot_dim=16, vdim=32, q_rank=64, kv_rank=64, window=150, mlp=all_chosen()),
                     pn.attention_layer(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, window=70),
                     pn.latent_layer(heads=2, dim=16, rot_dim=16, vdim=48, q_rank=32, kv_rank=32, window=33, mlp=pn.dense(96))], width=128)
    weights = write_model(tmp_path / "m", cfg, 22)
    tokens = tokens_of(cfg, 400, 11)
    runner = make_runner(tmp_path / "m", dtype, page_size=16, num_pages=64)
    ref = oracle(cfg, weights, tokens)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 400)]])["a"]
    cut = run_schedule(runner, {"b": tokens}, [[("b", 130)], [("b", 2)], [("b", 200)], [("b", 63)]] + [[("b", 1)] for _ in range(5)])["b"]
    assert_close(whole, ref, dtype, "whole")
    assert_close(cut, ref, dtype, "cut")


# -- keys just inside and just outside a window ---------------------------------------------------
def loud_pair(cfg: dict, weights: dict, key_token: int, query_token: int, wish: float = 20.0) -> None:
    """Change the embedding of ``key_token`` so that, in the one layer of ``cfg``, its key points
    where the query of ``query_token`` points in every head, and set the layer's score scale so
    that this pair's score (without the rotated part) is ``wish`` in the weakest head: wherever
    the key is visible to that query it takes nearly all of the softmax's weight."""
    layer, m = cfg["layers"][0], cfg["layers"][0]["mixer"]
    w = {k: v.double() for k, v in weights.items()}
    scale_in = cfg["embedding"]["scale"]
    h_q = w["embed"][query_token] * scale_in
    if layer["type"] == "attention":
        heads, kv_heads, dim, rot = m["heads"], m["kv_heads"], m["dim"], m["rot"]["dims"]
        q = (w["l0.mix.q"] @ h_q + w["l0.mix.q.b"]).view(kv_heads, heads // kv_heads, dim)
        target = q.mean(dim=1)                                   # what a key head's queries share
        target[:, :rot] = 0.0                                    # the rotated elements turn with the distance
        h_k = torch.linalg.lstsq(w["l0.mix.k"], (target.reshape(-1) - w["l0.mix.k.b"])[:, None]).solution[:, 0]
        weights["embed"][key_token] = (h_k / scale_in).to(weights["embed"].dtype)
        k = (w["l0.mix.k"] @ (weights["embed"][key_token].double() * scale_in) + w["l0.mix.k.b"]).view(kv_heads, dim)
        eps = cfg["norm"]["eps"]
        qn, kn = pn.rms(q, eps), pn.rms(k, eps)
        score = (qn[:, :, rot:] * kn[:, None, rot:]).sum(-1)
    else:
        heads, dim, rank = m["heads"], m["dim"], m["kv_rank"]
        eps = cfg["norm"]["eps"]
        c_q = pn.rms(w["l0.mix.dq"] @ h_q, eps) * w["l0.mix.dq.norm"]
        q = (w["l0.mix.uq"] @ c_q).view(heads, dim + m["rot_dim"])[:, :dim]
        latent = torch.linalg.lstsq(w["l0.mix.uk"], q.reshape(-1)[:, None]).solution[:, 0]
        # the shared rotated key part of this token is made zero: it would turn with the distance
        aim = torch.cat([latent / w["l0.mix.dkv.norm"], torch.zeros(m["rot_dim"], dtype=torch.float64)])
        h_k = torch.linalg.lstsq(w["l0.mix.dkv"], aim[:, None]).solution[:, 0]
        weights["embed"][key_token] = (h_k / h_k.abs().max() * 2.0 / scale_in).to(weights["embed"].dtype)
        down = w["l0.mix.dkv"][:rank] @ (weights["embed"][key_token].double() * scale_in)
        k = (w["l0.mix.uk"] @ (pn.rms(down, eps) * w["l0.mix.dkv.norm"])).view(heads, dim)
        score = (q * k).sum(-1)
    assert float(score.min()) > 0
    m["scale"] = wish / float(score.min())


def quiet_rotated_queries(cfg: dict, weights: dict) -> None:
    """A latent layer's sinks low and the rotated part of its queries small, so that the scores
    of the other keys stay well below the loud one's whatever their distance."""
    m = cfg["layers"][0]["mixer"]
    if cfg["layers"][0]["type"] != "latent_attention":
        return
    weights["l0.mix.sink"] = torch.full_like(weights["l0.mix.sink"], -1.0)
    rows = weights["l0.mix.uq"].view(m["heads"], m["dim"] + m["rot_dim"], -1)
    rows[:, m["dim"]:] *= 0.125


EDGE_LAYERS = {
    "attention": lambda window: pn.attention_layer(heads=4, kv_heads=2, dim=32, vdim=32, rot_dims=4, window=window, softcap=60.0, mlp=None),
    "attention_heads_of_64": lambda window: pn.attention_layer(heads=2, kv_heads=1, dim=64, vdim=64, rot_dims=8, window=window,
                                                               softcap=None, mlp=None),
    "attention_heads_of_128_capped": lambda window: pn.attention_layer(heads=4, kv_heads=2, dim=128, vdim=128, rot_dims=16, window=window,
                                                                       softcap=40.0, mlp=None),
    "latent": lambda window: pn.latent_layer(heads=2, dim=16, rot_dim=4, vdim=16, q_rank=32, kv_rank=72, window=window, mlp=None),
    "latent_sixteens": lambda window: pn.latent_layer(heads=4, dim=16, rot_dim=16, vdim=32, q_rank=64, kv_rank=112, window=window, mlp=None),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", (1, 2, 9, 16, 17, 70, 129))
@pytest.mark.parametrize("kind", sorted(EDGE_LAYERS))
def test_a_loud_key_just_inside_and_just_outside_the_window(tmp_path, kind, window, dtype):
    """One layer, one key that takes nearly all the weight of one query wherever it is visible.
    The query stands window - 1 tokens after the key (the last place that sees it) and once
    more a token later (the first that does not); in a whole prompt, in two portions cut
    between them, and decoded token by token; with pages of 4 and 16 tokens, so that the edge
    falls on, before and after a page border."""
    cfg = pn.config([EDGE_LAYERS[kind](window)], width=384 if "128" in kind else 192, vocab=40)
    key_token, query_token = 38, 39

    def change(weights):
        quiet_rotated_queries(cfg, weights)
        loud_pair(cfg, weights, key_token, query_token)

    weights = pn.random_weights(cfg, 23)
    change(weights)                       # sets the scale in cfg before the folder is written
    weights = write_model(tmp_path / "m", cfg, 23, change=change)
    at = 21                               # the key's place: not at a page's start
    length = at + window + 12
    tokens = tokens_of(cfg, length, 12, avoid=(key_token, query_token))
    tokens[at] = key_token
    inside, outside = at + window - 1, at + window
    if window > 1:
        tokens[inside] = query_token
    tokens[outside] = query_token
    ref = oracle(cfg, weights, tokens)
    plain = list(tokens)
    plain[at] = tokens[at + 1]
    without = oracle(cfg, weights, plain)
    difference = lambda i: float(((ref[i] - without[i]) ** 2).mean().sqrt() / (ref[i] ** 2).mean().sqrt())  # noqa: E731
    if window > 1:
        assert difference(inside) > 0.2, "the key inside the window decides the logits there"
    assert difference(outside) < 1e-9, "a token later nothing of it is left"
    for page_size in (4, 16):
        runner = make_runner(tmp_path / "m", dtype, page_size=page_size, num_pages=256 // page_size)
        whole = run_schedule(runner, {"a": tokens}, [[("a", length)]])["a"]
        cut = run_schedule(runner, {"b": tokens}, [[("b", at + 2)], [("b", inside - at - 2 + 1)], [("b", length - inside - 1)]]
                           if inside - at - 1 > 0 else [[("b", at + 1)], [("b", length - at - 1)]])["b"]
        head = max(1, at - 3)
        decoded = run_schedule(runner, {"c": tokens}, [[("c", head)]] + [[("c", 1)] for _ in range(length - head)])["c"]
        for got, what in ((whole, "prompt"), (cut, "portions"), (decoded, "decoded")):
            assert_close(got, ref, dtype, f"{what}, pages of {page_size}")
            for place in (inside, outside):
                assert_close(got[place : place + 1], ref[place : place + 1], dtype, f"{what} at {place}, pages of {page_size}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_token_far_back_reaches_late_logits_through_stacked_windows(tmp_path, dtype):
    """Three layers with windows of 16: a token 40 places back is out of every window's reach
    and still moves the last logits, through the layers between; one 46 places back cannot."""
    cfg = pn.config([pn.attention_layer(window=16, scale=0.6), pn.latent_layer(window=16, scale=0.5), pn.attention_layer(window=16, scale=0.6)])
    weights = write_model(tmp_path / "m", cfg, 24)
    tokens = tokens_of(cfg, 200, 13)
    last = len(tokens) - 1
    runner = make_runner(tmp_path / "m", dtype, page_size=16, num_pages=32)
    refs = {}
    for back in (0, 40, 46):
        ids = list(tokens)
        if back:
            ids[last - back] = (ids[last - back] + 1) % cfg["vocab"]
        refs[back] = oracle(cfg, weights, ids)
        for head in (len(ids), len(ids) - 10):
            got = run_schedule(runner, {"a": ids}, [[("a", head)]] + [[("a", 1)] for _ in range(len(ids) - head)])["a"]
            assert_close(got[-10:], refs[back][-10:], dtype, f"changed {back} back, {len(ids) - head} decoded")
    assert float((refs[40][last] - refs[0][last]).abs().max()) > 1e-6
    assert float((refs[46][last] - refs[0][last]).abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", (dict(), dict(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=32, kv_rank=48)), ids=("plain kernel", "tensor cores"))
def test_sinks_take_their_share(tmp_path, sizes, dtype):
    """Sinks from far below to far above the scores, one per head: the large ones take most of
    the weight (the head's output shrinks), the small ones none; counted once however the keys
    are split over blocks (decoding far into a long window splits them)."""
    cfg = pn.config([pn.latent_layer(window=300, mlp=None, **sizes)])
    heads = cfg["layers"][0]["mixer"]["heads"]

    def change(weights):
        weights["l0.mix.sink"] = torch.linspace(-30.0, 9.0, heads).to(torch.bfloat16)

    weights = write_model(tmp_path / "m", cfg, 26, change=change)
    tokens = tokens_of(cfg, 280, 14)
    ref = oracle(cfg, weights, tokens)
    flat = dict(weights)
    flat["l0.mix.sink"] = torch.full_like(weights["l0.mix.sink"], -1e4)
    assert float(((ref - oracle(cfg, flat, tokens)) ** 2).mean().sqrt() / (ref**2).mean().sqrt()) > 0.05
    runner = make_runner(tmp_path / "m", dtype, page_size=16, num_pages=32)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 280)]])["a"]
    decoded = run_schedule(runner, {"b": tokens}, [[("b", 250)]] + [[("b", 1)] for _ in range(30)])["b"]
    assert_close(whole, ref, dtype, "prompt")
    assert_close(decoded, ref, dtype, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(tmp_path, dtype):
    """Sequences of one to five tokens, alone and side by side, in slots and pages that hold an
    earlier request's keys: a first token sees itself (and the sink) and nothing else."""
    cfg = mixed_config(dtype)
    weights = write_model(tmp_path / "m", cfg, 25)
    runner = make_runner(tmp_path / "m", dtype, max_requests=4, num_pages=24)
    warm = {key: tokens_of(cfg, 12, 40 + i) for i, key in enumerate("wxyz")}
    run_schedule(runner, warm, [[(key, 12) for key in warm]])
    requests = {key: tokens_of(cfg, n, 30 + n) for key, n in (("a", 1), ("b", 2), ("c", 3), ("d", 5))}
    got = run_schedule(runner, requests, [[("a", 1), ("b", 1), ("c", 3), ("d", 2)], [("b", 1), ("d", 3)]])
    for key, tokens in requests.items():
        assert_close(got[key], oracle(cfg, weights, tokens), dtype, f"request {key}")


# -- parts alone -------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("experts, top, groups, tokens, ff", (
    (6, 2, (3, 2), 150, 32), (12, 2, (2, 1), 300, 96), (8, 4, (4, 2), 300, 48), (6, 2, None, 33, 24), (4, 2, (4, 3), 40, 16),
    (16, 3, (4, 2), 700, 64), (5, 1, (1, 1), 5, 40), (30, 6, (10, 3), 64, 16), (12, 3, (3, 1), 90, 20)))
def test_routed_feed_forward_alone(experts, top, groups, tokens, ff, dtype):
    """The part alone against a loop over tokens and experts: sigmoid scores, groups worth the
    sum of their two largest scores (or of their one), weights as the scores are, units without
    a gate and with the square of relu.  Tokens whose choice is not clear (of groups or of
    experts) are left out."""
    from forge_engine_b200.config.specs import DenseMLPSpec, RoutedMLPSpec
    from forge_engine_b200.parts.base import BuildContext, build_part

    gen = torch.Generator().manual_seed(experts * 10 + top)
    width = 48
    mlp = pn.routed(experts=experts, top=top, ff=ff, groups=groups)
    cfg = pn.config([pn.latent_layer(mlp=mlp)], width=width)
    weights = {name[len("l0.mlp."):]: t for name, t in pn.random_weights(cfg, 7).items() if name.startswith("l0.mlp.")}
    weights["router"] = (3.0 * torch.randn(experts, width, generator=gen) / math.sqrt(width)).to(torch.bfloat16)
    x = torch.randn(tokens, width, generator=gen).to(torch.bfloat16)
    chosen = []
    want = pn.routed_feed_forward(x.double(), {"l0.mlp." + k: v.double() for k, v in weights.items()}, "l0.mlp.", mlp, chosen_out=chosen)
    scores = torch.sigmoid(x.double() @ weights["router"].double().T)
    count, keep = groups or (1, 1)
    size = experts // count
    worth = scores.view(tokens, count, size).sort(dim=-1, descending=True).values[..., :2].sum(-1).sort(dim=-1, descending=True).values
    clear = torch.ones(tokens, dtype=torch.bool)
    if keep < count:
        clear &= (worth[:, keep - 1] - worth[:, keep]) > 2e-3
    for t in range(tokens):
        kept = {e // size for e in chosen[t]}
        open_groups = sorted(range(count), key=lambda g: -float(scores[t].view(count, size)[g].sort(descending=True).values[:2].sum()))[:keep]
        assert kept <= set(open_groups)
        allowed = sorted((float(scores[t, e]) for e in range(experts) if e // size in open_groups), reverse=True)
        if top < len(allowed) and allowed[top - 1] - allowed[top] <= 2e-3:
            clear[t] = False
    assert int(clear.sum()) >= tokens // 2
    unit = DenseMLPSpec(width, ff, "relu2", bias=False, rename=(("up_proj.weight", "up"), ("down_proj.weight", "down")))
    spec = RoutedMLPSpec(width, experts, top, unit, shared=None, score="sigmoid", renormalise=False, weight_on="output",
                         groups=groups, group_score="top2")
    ctx = BuildContext(dtype=dtype, device=torch.device("cuda"), status=torch.zeros(1, dtype=torch.int32, device="cuda"))
    part = build_part(spec, {k: v.to(dtype).cuda() for k, v in weights.items()}, ctx)
    assert part.fused == (dtype == torch.bfloat16 and ff % 8 == 0)
    for _ in range(2):      # the second call finds the counts as the first left them
        got = part.forward(x.to(dtype).cuda()).float().cpu()
    assert int(ctx.status.item()) == 0
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert float((got[clear] - want[clear].float()).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    assert int(part.counts.abs().sum()) == 0


def test_a_group_of_two_strong_experts_beats_one_stronger():
    """Where the largest single score and the largest sum of two lie in different groups, the
    sum decides: made so by the router's rows, with margins far above rounding."""
    from forge_engine_b200.ops import native

    logits = torch.full((3, 6), -4.0)
    logits[0, 0], logits[0, 3], logits[0, 4] = 3.0, 1.0, 1.2      # group 0 holds the largest, group 1 the best pair
    logits[1, 5], logits[1, 0] = 0.5, 0.4                         # here the single large one wins: 0.62 + 0.02 > 0.60 + 0.02
    logits[2, 2], logits[2, 3] = 2.0, 2.0                         # equal groups: the lower index
    want = [{3, 4}, {5, 3}, {2, 0}]
    experts, top = 6, 2
    counts = torch.zeros(experts + 1, dtype=torch.int32, device="cuda")
    max_tiles = native.moe_max_tiles(3 * top, experts, 0)
    ints = torch.empty(4 * 3 * top + experts + 2 + 2 * max_tiles, dtype=torch.int32, device="cuda")
    weight = torch.empty(3 * top, dtype=torch.float32, device="cuda")
    plan = native.moe_route(logits.cuda(), experts, top, False, False, counts, ints, weight, max_tiles, groups=(2, 1), group_top2=True)
    got = plan["slot_expert"].cpu().view(3, top).tolist()
    for row, (mine, ref) in enumerate(zip(got, want)):
        assert set(mine) == ref, f"token {row}: {mine}"           # equal scores: the lower index
    scores = torch.sigmoid(logits)
    for row in range(3):
        for k in range(top):
            assert abs(float(weight[row * top + k]) - float(scores[row, got[row][k]])) < 1e-6


# -- generation through the engine's own entry points ------------------------------------------------
def test_greedy_generation_through_engine_and_scheduler(tmp_path):
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine

    cfg = mixed_config()
    weights = write_model(tmp_path / "m", cfg, 18)
    prompts = [tokens_of(cfg, n, 20 + n) for n in (3, 26, 11, 1, 17)]
    engine = Engine.from_pretrained(
        tmp_path / "m",
        engine_config=EngineConfig(max_new_tokens=7, dtype="float32"),
        scheduler_config=SchedulerConfig(max_requests=3, max_batch_size=3, token_budget=12, block_size=4,
                                         block_capacity=96, chunk_size=8),
    )
    outputs = engine.generate(prompts)
    engine.runner.cache.check_consistency()
    assert engine.runner.cache.live_requests == 0
    for prompt, output in zip(prompts, outputs):
        assert len(output) == 7
        ids = list(prompt)
        for token in output:
            ref = oracle(cfg, weights, ids)[-1]
            top = torch.topk(ref, 2).values
            assert token == int(ref.argmax()) or float(top[0] - top[1]) < 1e-3
            ids.append(token)


def test_generate_command(tmp_path, capsys):
    from forge_engine_b200.cli import main

    cfg = pn.config([pn.latent_layer(), pn.attention_layer(mlp=pn.routed()), pn.latent_layer(mlp=None)])
    weights = write_model(tmp_path / "m", cfg, 19)
    prompt = tokens_of(cfg, 9, 1)
    code = main(["generate", "--model", str(tmp_path / "m"), "--prompt-ids", ",".join(map(str, prompt)),
                 "--max-new-tokens", "4", "--dtype", "float32", "--block-size", "4", "--block-capacity", "32"])
    assert code == 0
    printed = [int(t) for t in capsys.readouterr().out.strip().splitlines()[-1].split(",")]
    assert printed == pn.greedy_generate(cfg, weights, prompt, 4)


def test_random_weights_model_steps():
    """Seeded random weights for a configuration (what the benchmark uses): the model is
    assembled without a checkpoint and its logits do not depend on how the prompt was cut."""
    from forge_engine_b200.engine import ModelRunner

    cfg = mixed_config("bfloat16")
    runner = ModelRunner.from_random(cfg, 5, dtype="bfloat16", page_size=16, num_pages=32, max_requests=2, std=0.05)
    tokens = tokens_of(cfg, 40, 3)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 40)]])["a"]
    cut = run_schedule(runner, {"b": tokens}, [[("b", 23)], [("b", 16)], [("b", 1)]])["b"]
    assert torch.isfinite(whole).all()
    assert float((whole - cut).abs().max()) <= 0.05 * max(1.0, float(whole.abs().max()))
