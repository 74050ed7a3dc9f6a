"""The Zabutar design in the engine against the plain implementation of ``plain_zabutar.py``:
every mechanism alone, whole prompts against portions and token-by-token decoding, unequal
batches, reused pages and slots, far keys and the edges of the distance buckets, the first
tokens of a sequence (the convolution's zeros), other sizes, generation."""

from __future__ import annotations

import json
import math

import pytest
import torch
from safetensors.torch import save_file

import plain_zabutar as pz

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


# -- helpers --------------------------------------------------------------------------------
def write_model(folder, cfg: dict, seed: int, change=None) -> dict:
    weights = pz.random_weights(cfg, seed)
    if change is not None:
        change(weights)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(pz.written(cfg)))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return weights


def make_runner(folder, dtype: str, page_size=4, num_pages=96, max_requests=4, use_graphs=True):
    from forge_engine_b200.engine import ModelRunner

    return ModelRunner.from_folder(folder, dtype=dtype, page_size=page_size, num_pages=num_pages,
                                   max_requests=max_requests, use_graphs=use_graphs)


def tokens_of(cfg: dict, length: int, seed: int) -> list:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (length,), generator=gen).tolist()


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
    return pz.forward(cfg, weights, tokens)


def all_chosen():
    """A routed feed-forward in which every expert of the kept groups is chosen, so that
    nothing rests on a close call of the router (which bfloat16 rounding decides otherwise)."""
    return pz.routed(experts=3, identity=1, top=4, ff=32, groups=(1, 1), scale=1.5, shared_ff=40)


def routed_for(dtype: str, **kwargs):
    return pz.routed(**kwargs) if dtype == "float32" else all_chosen()


def mixed_config(dtype: str = "float32"):
    """All mechanisms in one model: recurrent layers with dense and routed feed-forwards, an
    attention layer, a layer without feed-forward, and a layer that reads another's keys and
    values.  Routers that choose are compared in 32-bit (a close call decided the other way
    by bfloat16 rounding changes a token's logits far beyond rounding) and, in bfloat16, on
    the part alone where the margins are known."""
    return pz.config([
        pz.recurrent_layer(),
        pz.attention_layer(mlp=routed_for(dtype)),
        pz.recurrent_layer(heads=2, dim=16, vdim=8, mlp=routed_for(dtype, top=3, groups=(2, 1), experts=6, identity=2)),
        pz.attention_layer(heads=2, kv_heads=1, dim=32, vdim=16, bias_rows=8, bias_max=17.5, mlp=None),
        pz.attention_layer(kv_from=1),
        pz.recurrent_layer(mlp=None),
    ])


# -- every mechanism alone --------------------------------------------------------------------
SINGLE = {
    "recurrence_dense": [pz.recurrent_layer()],
    "recurrence_no_ff": [pz.recurrent_layer(mlp=None)],
    "recurrence_odd_sizes": [pz.recurrent_layer(heads=3, dim=10, vdim=12)],
    "recurrence_one_head": [pz.recurrent_layer(heads=1, dim=64, vdim=64)],
    "attention_dense": [pz.attention_layer()],
    "attention_no_ff": [pz.attention_layer(mlp=None)],
    "attention_odd_sizes": [pz.attention_layer(heads=3, kv_heads=1, dim=12, vdim=20)],
    "attention_heads_of_64": [pz.attention_layer(heads=2, kv_heads=2, dim=64, vdim=64, bias_rows=32, bias_max=100)],
    "attention_wide_values": [pz.attention_layer(heads=2, kv_heads=1, dim=16, vdim=48)],
    "attention_two_rows": [pz.attention_layer(bias_rows=2, bias_max=9)],
    "attention_shared_keys": [pz.attention_layer(), pz.attention_layer(kv_from=0, mlp=None)],
    "routed": [pz.recurrent_layer(mlp=pz.routed())],
    "routed_one_no_shared": [pz.recurrent_layer(mlp=pz.routed(top=1, shared_ff=None))],
    "routed_no_identity": [pz.attention_layer(mlp=pz.routed(experts=6, identity=0, top=2))],
    "routed_one_group": [pz.attention_layer(mlp=pz.routed(experts=4, identity=3, top=3, groups=(1, 1)))],
    "routed_all": [pz.recurrent_layer(mlp=all_chosen())],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    if dtype == "bfloat16" and name.startswith("routed") and name != "routed_all":
        pytest.skip("routers that choose are compared in 32-bit and on the part alone")
    cfg = pz.config(SINGLE[name])
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
    tokens = tokens_of(cfg, 21, 6)
    want = []
    pz.forward(cfg, weights, tokens, layers_out=want)
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
    """Portions down to two tokens (and one): shorter than the convolution's reach, so the
    state's rows and the portion's own meet inside one token's taps."""
    cfg = mixed_config(dtype)
    cfg["canon"]["taps"] = 4
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
    """Two slots and a pool that holds two requests at most: later requests get the pages,
    the recurrent state and the convolution's rows of earlier ones, which must read as new."""
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
    """A short prompt, then far more single tokens than the distance buckets reach or a page
    holds; the decode steps are replayed from captured graphs."""
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
    and replayed (filler entries pad them to their bucket, with the cache's null slot as their
    state).  Logits at every entry's last token against the plain implementation."""
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
    "one_tap": dict(layers=[pz.recurrent_layer(), pz.attention_layer()], taps=1),
    "two_taps": dict(layers=[pz.recurrent_layer(), pz.attention_layer(mlp=None)], taps=2),
    "eight_taps": dict(layers=[pz.attention_layer(), pz.recurrent_layer(mlp=None)], taps=8),
    "narrow": dict(layers=[pz.recurrent_layer(heads=1, dim=4, vdim=4), pz.attention_layer(heads=1, kv_heads=1, dim=8, vdim=8)],
                   width=20, vocab=11),
    "width_not_in_eights": dict(layers=[pz.recurrent_layer(heads=2, dim=6, vdim=10), pz.attention_layer(mlp=pz.routed())],
                                width=36),
    "every_head_its_own_keys": dict(layers=[pz.attention_layer(heads=4, kv_heads=4)]),
    "one_key_head": dict(layers=[pz.attention_layer(heads=6, kv_heads=1, dim=32, vdim=32)]),
    "wide_state": dict(layers=[pz.recurrent_layer(heads=2, dim=96, vdim=128)], width=128),
    "long_state_rows": dict(layers=[pz.recurrent_layer(heads=1, dim=200, vdim=24)]),
    "attention_first_shared_last": dict(layers=[pz.attention_layer(dim=32, vdim=48), pz.recurrent_layer(), pz.recurrent_layer(),
                                                pz.attention_layer(dim=32, vdim=48, kv_from=0, mlp=pz.routed(top=1))]),
    "two_sources": dict(layers=[pz.attention_layer(), pz.attention_layer(heads=2, kv_heads=2, dim=8, vdim=8),
                                pz.attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, kv_from=1), pz.attention_layer(kv_from=0)]),
    "scale_one_eps_large": dict(layers=[pz.attention_layer(scale=1.0), pz.recurrent_layer()], eps=0.5),
    "top_equals_experts": dict(layers=[pz.recurrent_layer(mlp=pz.routed(experts=4, identity=0, top=4, groups=(2, 2), scale=1.0))]),
    "identity_only_choice": dict(layers=[pz.recurrent_layer(mlp=pz.routed(experts=1, identity=3, top=2, groups=(2, 1)))]),
}


@pytest.mark.parametrize("name", sorted(OTHER))
def test_other_sizes_and_values_that_are_one_or_equal(tmp_path, name):
    options = dict(OTHER[name])
    cfg = pz.config(options.pop("layers"), **options)
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
    tensor-core attention kernel, with steps long enough for several row tiles."""
    cfg = pz.config([pz.recurrent_layer(heads=2, dim=32, vdim=64, mlp=all_chosen()),
                     pz.attention_layer(heads=4, kv_heads=2, dim=64, vdim=64, bias_rows=16, bias_max=300),
                     pz.attention_layer(heads=4, kv_heads=2, dim=64, vdim=64, bias_rows=6, bias_max=33, kv_from=1)], width=128)
    weights = write_model(tmp_path / "m", cfg, 22)
    tokens = tokens_of(cfg, 400, 11)
    runner = make_runner(tmp_path / "m", dtype, page_size=16, num_pages=64)
    ref = oracle(cfg, weights, tokens)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 400)]])["a"]
    cut = run_schedule(runner, {"b": tokens}, [[("b", 130)], [("b", 2)], [("b", 200)], [("b", 63)]] + [[("b", 1)] for _ in range(5)])["b"]
    assert_close(whole, ref, dtype, "whole")
    assert_close(cut, ref, dtype, "cut")


# -- keys far away and at the edges of the distance buckets -------------------------------------------
def loud_bias(weights: dict) -> None:
    """A bias table whose rows differ by much more than any score: a key read with a
    neighbouring row's bias changes the output far beyond rounding."""
    for name in weights:
        if name.endswith("mix.rel"):
            rows = weights[name].shape[0]
            weights[name] = (4.0 * torch.randn(weights[name].shape, generator=torch.Generator().manual_seed(rows))).to(torch.bfloat16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim", ((2, 1, 16), (4, 2, 64)), ids=("heads of 16", "heads of 64"))
@pytest.mark.parametrize("rows, far", ((12, 40), (8, 17.5), (30, 140), (4, 3), (6, 250)))
def test_keys_at_the_edges_of_the_distance_buckets(tmp_path, rows, far, dtype, heads, kv_heads, dim):
    """Every distance up to well past ``far`` occurs, in a prompt (whole and in two portions)
    and for decoded tokens, with a table that makes a wrong row show; the page size is not a
    divisor of any bucket's edge.  Heads of 64 take the tensor-core prompt kernel in bfloat16."""
    cfg = pz.config([pz.attention_layer(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, bias_rows=rows, bias_max=far, mlp=None)], width=32)
    weights = write_model(tmp_path / "m", cfg, 23, change=loud_bias)
    length = max(40, min(int(far * 1.3) + 12, 330))
    tokens = tokens_of(cfg, length, 12)
    ref = oracle(cfg, weights, tokens)
    runner = make_runner(tmp_path / "m", dtype, page_size=4, num_pages=96)
    whole = run_schedule(runner, {"a": tokens}, [[("a", length)]])["a"]
    head = length - 20
    decoded = run_schedule(runner, {"b": tokens}, [[("b", head)]] + [[("b", 1)] for _ in range(20)])["b"]
    cut = run_schedule(runner, {"c": tokens}, [[("c", 13)], [("c", length - 13)]])["c"]
    assert_close(whole, ref, dtype, "prompt")
    assert_close(decoded, ref, dtype, "decoded")
    assert_close(cut, ref, dtype, "two portions")
    # the table is what decides: with a flat table the logits are far from these
    flat = dict(weights)
    flat["l0.mix.rel"] = torch.zeros_like(weights["l0.mix.rel"])
    other = oracle(cfg, flat, tokens)
    assert float(((ref - other) ** 2).mean().sqrt() / (ref**2).mean().sqrt()) > 0.05


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim", (16, 64))
@pytest.mark.parametrize("new_tokens", (1, 0))
def test_a_far_key_among_hundreds(tmp_path, new_tokens, dtype, dim):
    """One early key is made to stand out (its token's embedding and the last token's are
    scaled so that their score towers over the rest) and the table's last row favours far keys:
    the late logits rest on a key 300 tokens back, in a prompt and when decoding."""
    cfg = pz.config([pz.attention_layer(heads=2, kv_heads=1, dim=dim, vdim=dim, bias_rows=8, bias_max=64, mlp=None)],
                    width=32, vocab=50)

    def change(weights):
        weights["l0.mix.rel"][-1] = 6.0
        weights["l0.mix.rel"][:-1] = -2.0

    weights = write_model(tmp_path / "m", cfg, 24, change=change)
    tokens = tokens_of(cfg, 320, 13)
    other = list(tokens)
    other[7] = (tokens[7] + 1) % cfg["vocab"]
    runner = make_runner(tmp_path / "m", dtype, page_size=16, num_pages=48)
    refs = []
    for ids in (tokens, other):
        ref = oracle(cfg, weights, ids)
        refs.append(ref)
        head = len(ids) - 10 * new_tokens
        got = run_schedule(runner, {"a": ids}, [[("a", head)]] + [[("a", 1)] for _ in range(len(ids) - head)])["a"]
        assert_close(got[-10:], ref[-10:], dtype, "late logits")
    late = slice(310, 320)
    assert float(((refs[0][late] - refs[1][late]) ** 2).mean().sqrt() / (refs[0][late] ** 2).mean().sqrt()) > 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_first_tokens_of_a_sequence(tmp_path, dtype):
    """Sequences of one to five tokens, alone and side by side, with five taps: every token
    reads zeros before the sequence's start, never a neighbour's rows or an earlier request's."""
    cfg = mixed_config(dtype)
    cfg["canon"]["taps"] = 5
    weights = write_model(tmp_path / "m", cfg, 25)
    runner = make_runner(tmp_path / "m", dtype, max_requests=4)
    # a first round leaves rows in every slot's state
    warm = {key: tokens_of(cfg, 12, 40 + i) for i, key in enumerate("wxyz")}
    run_schedule(runner, warm, [[(key, 12) for key in warm]])
    requests = {key: tokens_of(cfg, n, 30 + n) for key, n in (("a", 1), ("b", 2), ("c", 3), ("d", 5))}
    got = run_schedule(runner, requests, [[("a", 1), ("b", 1), ("c", 3), ("d", 2)], [("b", 1), ("d", 3)]])
    for key, tokens in requests.items():
        assert_close(got[key], oracle(cfg, weights, tokens), dtype, f"request {key}")


# -- kernels and parts alone -----------------------------------------------------------------------
def cuda_batch(counts, slots):
    """cu_tokens, token_entry and slots of a step whose entries bring ``counts`` tokens."""
    cu = [0]
    for n in counts:
        cu.append(cu[-1] + n)
    entry = [i for i, n in enumerate(counts) for _ in range(n)]
    as_int = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")  # noqa: E731
    return as_int(cu), as_int(entry), as_int(slots)


SHORT_ENTRIES = {0: [19, 1, 2], 3: [1, 37, 1], 1: [2, 3, 40]}
# entries long enough for the chunk-parallel kernels beside short ones: a chunk's length and
# its neighbours, one token over a chunk, several chunks, a last chunk of one token
LONG_ENTRIES = {0: [300, 1, 129], 3: [1, 128, 70], 1: [64, 127, 257]}


@pytest.mark.parametrize("lengths", (SHORT_ENTRIES, LONG_ENTRIES), ids=("short", "long"))
@pytest.mark.parametrize("heads, dk, dv", ((4, 8, 16), (3, 10, 12), (1, 64, 64), (2, 96, 128), (1, 200, 24), (5, 4, 4), (2, 56, 24)))
def test_gated_recurrence_kernel(heads, dk, dv, lengths):
    """Entries of unequal lengths, carried over three calls from the state rows, against a
    loop over time; a slot that is zeroed and used again starts from nothing."""
    from forge_engine_b200.ops import native

    gen = torch.Generator().manual_seed(heads * 100 + dk)
    qk, v = heads * dk, heads * dv
    lower = torch.rand(qk, generator=gen) * 0.9
    f_bias = torch.randn(qk, generator=gen)
    norm = 1.0 + 0.2 * torch.randn(dv, generator=gen)
    eps = 1e-5
    state = torch.zeros(5, heads, dk, dv, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    history = {slot: [] for slot in lengths}
    for call in range(3):
        counts = [lengths[slot][call] for slot in lengths]
        n = sum(counts)
        proj = torch.randn(n, 2 * qk + v + 3, generator=gen)
        cu, _, slots = cuda_batch(counts, list(lengths))
        out = torch.empty(n, v, device="cuda")
        native.gated_recurrence(proj.cuda(), 3, 3 + qk, 3 + 2 * qk, f_bias.cuda(), lower.cuda(), norm.cuda(), eps, state,
                                slots, cu, out, len(counts), status, max_new=max(counts))
        at = 0
        for slot, count in zip(lengths, counts):
            history[slot].append((proj[at : at + count].double(), out[at : at + count].cpu()))
            at += count
    assert int(status.item()) == 0
    for slot, pieces in history.items():
        rows = torch.cat([p for p, _ in pieces])
        got = torch.cat([o for _, o in pieces])
        q = torch.nn.functional.silu(rows[:, 3 : 3 + qk]).view(-1, heads, dk)
        f = (lower.double() + (1 - lower.double()) * torch.sigmoid(rows[:, 3 + qk : 3 + 2 * qk] + f_bias.double())).view(-1, heads, dk)
        val = rows[:, 3 + 2 * qk : 3 + 2 * qk + v].view(-1, heads, dv)
        s = torch.zeros(heads, dk, dv, dtype=torch.float64)
        want = torch.empty(rows.shape[0], heads, dv, dtype=torch.float64)
        for t in range(rows.shape[0]):
            s = f[t][:, :, None] * s + (1 - f[t])[:, :, None] * val[t][:, None, :]
            want[t] = torch.einsum("hdv,hd->hv", s, q[t])
        want = pz.rms(want, eps) * norm.double()
        assert float((got - want.reshape(-1, v).float()).abs().max()) <= 2e-4 * max(1.0, float(want.abs().max()))
        assert float((state[slot].cpu() - s.float()).abs().max()) <= 1e-4 * max(1.0, float(s.abs().max()))
    assert float(state[[2, 4]].abs().max()) == 0.0       # rows of no entry are not touched


@pytest.mark.parametrize("taps", (1, 2, 3, 4, 5, 8))
@pytest.mark.parametrize("out_dtype", (torch.float32, torch.bfloat16))
def test_causal_convolution_kernel(taps, out_dtype):
    """Entries shorter and longer than the taps reach, over four calls: the rows before an
    entry's first token come from the state, zeros at a sequence's start."""
    from forge_engine_b200.ops import native

    gen = torch.Generator().manual_seed(taps)
    width = 40
    w = 0.5 * torch.randn(width, taps, generator=gen)
    state = torch.zeros(4, 2, max(taps - 1, 1), width, device="cuda")
    state[:, 0] = 7.0          # the other sublayer's rows: never read, never written
    lengths = {2: [1, 2, 9, 1], 0: [13, 1, 1, 2], 1: [3, 3, 1, 30]}
    seen = {slot: [] for slot in lengths}
    for call in range(4):
        counts = [lengths[slot][call] for slot in lengths]
        n = sum(counts)
        y = torch.randn(n, width, generator=gen)
        cu, entry, slots = cuda_batch(counts, list(lengths))
        out = torch.empty(n, width, dtype=out_dtype, device="cuda")
        native.causal_conv_state(y.cuda(), w.t().contiguous().cuda(), state[:, 1] if taps > 1 else None, slots, cu, entry, out,
                                 len(counts))
        at = 0
        for slot, count in zip(lengths, counts):
            seen[slot].append((y[at : at + count], out[at : at + count].float().cpu()))
            at += count
    for slot, pieces in seen.items():
        want = pz.short_convolution(torch.cat([y for y, _ in pieces]).double(), w.double())
        got = torch.cat([o for _, o in pieces])
        tol = 1e-5 if out_dtype == torch.float32 else 2e-2
        assert float((got - want.float()).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    assert float((state[:, 0] - 7.0).abs().max()) == 0.0


def test_activation_and_double_norm_kernels():
    from forge_engine_b200.ops import native

    gen = torch.Generator().manual_seed(3)
    x = 3.0 * torch.randn(33, 50, generator=gen)
    bias = torch.randn(50, generator=gen)
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.8, dtype=torch.float64)
    out = torch.empty(33, 50, device="cuda")
    native.bias_xielu(x.cuda(), bias.cuda(), out, float(pz.softplus(p)), 0.5 + float(pz.softplus(q)))
    want = pz.xielu(x.double() + bias.double(), p, q)
    assert float((out.cpu() - want.float()).abs().max()) <= 1e-5 * float(want.abs().max())
    # residual += norm_b(update); out = norm(residual), on all rows and on mapped rows
    res = torch.randn(9, 50, generator=gen)
    upd = 4.0 * torch.randn(9, 50, generator=gen)
    wb, wn = torch.randn(50, generator=gen), torch.randn(50, generator=gen)
    total = res.double() + pz.rms(upd.double(), 1e-3) * wb.double()
    want = pz.rms(total, 1e-6) * wn.double()
    stream = res.clone().cuda()
    rows = torch.tensor([7, 2], dtype=torch.int32, device="cuda")
    mapped = torch.empty(2, 50, device="cuda")
    native.add_normed_rmsnorm(stream, upd.cuda(), wb.cuda(), wn.cuda(), mapped, 1e-3, 1e-6, row_map=rows, write_residual=False)
    assert float((stream.cpu() - res).abs().max()) == 0.0
    assert float((mapped.cpu() - want[[7, 2]].float()).abs().max()) <= 1e-5 * float(want.abs().max())
    out = torch.empty(9, 50, device="cuda")
    native.add_normed_rmsnorm(stream, upd.cuda(), wb.cuda(), wn.cuda(), out, 1e-3, 1e-6)
    assert float((stream.cpu() - total.float()).abs().max()) <= 1e-5 * float(total.abs().max())
    assert float((out.cpu() - want.float()).abs().max()) <= 1e-5 * float(want.abs().max())


@pytest.mark.parametrize("width", (40, 50, 37))
@pytest.mark.parametrize("taps", (1, 2, 4, 8))
@pytest.mark.parametrize("out_dtype", (torch.float32, torch.bfloat16))
def test_norm_and_convolution_in_one_launch(taps, out_dtype, width):
    """Steps in which every entry brings one token: the norms, the sum and the convolution in
    one launch give bit for bit what the two kernels give one after the other, in the results,
    the stream and the state, over several steps and with slots in any order; and both follow
    the plain functions."""
    from forge_engine_b200.ops import native

    gen = torch.Generator().manual_seed(taps * 100 + width)
    w = 0.5 * torch.randn(width, taps, generator=gen)
    taps_weight = w.t().contiguous().cuda()
    wb, wn = torch.randn(width, generator=gen), torch.randn(width, generator=gen)
    order = [3, 0, 2]
    slots = torch.tensor(order, dtype=torch.int32, device="cuda")
    cu, entry, _ = cuda_batch([1, 1, 1], order)
    states = [torch.zeros(4, 2, max(taps - 1, 1), width, device="cuda") for _ in range(2)]
    streams = [torch.randn(3, width, generator=gen).cuda()] * 2
    streams = [streams[0].clone(), streams[1].clone()]
    rows_of = {slot: [] for slot in order}
    for step in range(taps + 2):
        upd = (3.0 * torch.randn(3, width, generator=gen)).cuda()
        before = streams[0].cpu().double()
        fused = torch.empty(3, width, dtype=out_dtype, device="cuda")
        native.add_normed_rmsnorm(streams[0], upd, wb.cuda(), wn.cuda(), fused, 1e-3, 1e-6,
                                  conv=(taps_weight, states[0][:, 1] if taps > 1 else None, slots))
        y = torch.empty(3, width, device="cuda")
        native.add_normed_rmsnorm(streams[1], upd, wb.cuda(), wn.cuda(), y, 1e-3, 1e-6)
        apart = torch.empty(3, width, dtype=out_dtype, device="cuda")
        native.causal_conv_state(y, taps_weight, states[1][:, 1] if taps > 1 else None, slots, cu, entry, apart, 3)
        assert torch.equal(fused, apart) and torch.equal(streams[0], streams[1]) and torch.equal(states[0], states[1])
        total = before + pz.rms(upd.cpu().double(), 1e-3) * wb.double()
        normed = pz.rms(total, 1e-6) * wn.double()
        for i, slot in enumerate(order):
            rows_of[slot].append((normed[i], fused[i].float().cpu()))
    for slot, pieces in rows_of.items():
        want = pz.short_convolution(torch.stack([y for y, _ in pieces]), w.double())
        got = torch.stack([o for _, o in pieces])
        tol = 1e-5 if out_dtype == torch.float32 else 2e-2
        assert float((got - want.float()).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    assert float(states[0][:, 0].abs().max()) == 0.0 and float(states[0][1].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("experts, identity, top, groups, tokens, ff", (
    (5, 1, 2, (3, 2), 150, 32), (9, 3, 4, (4, 2), 300, 48), (6, 0, 2, (1, 1), 33, 24), (1, 3, 2, (2, 1), 40, 16),
    (12, 4, 3, (4, 2), 700, 64), (4, 2, 1, (6, 1), 5, 40), (30, 2, 6, (8, 3), 64, 16)))
def test_routed_feed_forward_alone(experts, identity, top, groups, tokens, ff, dtype):
    """The part alone against a loop over tokens and experts: softmax over all outputs, the
    correction in the choice only, groups (choice scores can be negative: the correction is
    made large), identity experts, the weights' floor and scale, the shared unit.  Tokens whose
    choice is not clear (of groups or of experts) are left out."""
    from forge_engine_b200.config.specs import GatedMLPSpec, RoutedMLPSpec
    from forge_engine_b200.parts.base import BuildContext, build_part

    gen = torch.Generator().manual_seed(experts * 10 + identity)
    width, scale = 48, 1.75
    mlp = pz.routed(experts=experts, identity=identity, top=top, ff=ff, groups=groups, scale=scale, shared_ff=32)
    cfg = pz.config([pz.recurrent_layer(mlp=mlp)], width=width)
    weights = {name[len("l0.mlp."):]: t for name, t in pz.random_weights(cfg, 7).items() if name.startswith("l0.mlp.")}
    outputs = experts + identity
    weights["router"] = (3.0 * torch.randn(outputs, width, generator=gen) / math.sqrt(width)).to(torch.bfloat16)
    weights["correction"] = (0.3 * torch.randn(outputs, generator=gen) - 0.2).to(torch.bfloat16)
    x = torch.randn(tokens, width, generator=gen).to(torch.bfloat16)
    want = pz.routed_feed_forward(x.double(), {"l0.mlp." + k: v.double() for k, v in weights.items()}, "l0.mlp.", mlp)
    # clear choices: margins between the groups at the edge and between the experts at the edge
    choice = torch.softmax(x.double() @ weights["router"].double().T, dim=-1) + weights["correction"].double()
    assert bool((choice < 0).any())
    size = outputs // groups[0]
    marks = choice.view(tokens, groups[0], size).max(dim=-1).values.sort(dim=-1, descending=True).values
    clear = torch.ones(tokens, dtype=torch.bool)
    if groups[1] < groups[0]:
        clear &= (marks[:, groups[1] - 1] - marks[:, groups[1]]) > 2e-3
    for t in range(tokens):
        kept = sorted(range(groups[0]), key=lambda g: -float(choice[t].view(groups[0], size)[g].max()))[: groups[1]]
        allowed = sorted((float(choice[t, e]) for e in range(outputs) if e // size in kept), reverse=True)
        if top < len(allowed) and allowed[top - 1] - allowed[top] <= 2e-3:
            clear[t] = False
    assert int(clear.sum()) >= tokens // 2
    unit = dict(rename=(("gate_proj.weight", "gate"), ("up_proj.weight", "up"), ("down_proj.weight", "down")))
    spec = RoutedMLPSpec(width, experts, top, GatedMLPSpec(width, ff, "silu", **unit), shared=GatedMLPSpec(width, 32, "silu", **unit),
                         score="softmax", renormalise=True, weight_on="output", identity=identity, correction=True,
                         groups=groups, renorm_floor=1e-20, weight_scale=scale)
    ctx = BuildContext(dtype=dtype, device=torch.device("cuda"), status=torch.zeros(1, dtype=torch.int32, device="cuda"))
    part = build_part(spec, {k: v.to(dtype).cuda() for k, v in weights.items()}, ctx)
    assert part.fused == (dtype == torch.bfloat16 and ff % 16 == 0)
    for _ in range(2):      # the second call finds the counts as the first left them
        got = part.forward(x.to(dtype).cuda()).float().cpu()
    assert int(ctx.status.item()) == 0
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert float((got[clear] - want[clear].float()).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    assert int(part.counts.abs().sum()) == 0


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

    cfg = pz.config([pz.recurrent_layer(), pz.attention_layer(mlp=pz.routed()), pz.attention_layer(kv_from=1, mlp=None)])
    weights = write_model(tmp_path / "m", cfg, 19)
    prompt = tokens_of(cfg, 9, 1)
    code = main(["generate", "--model", str(tmp_path / "m"), "--prompt-ids", ",".join(map(str, prompt)),
                 "--max-new-tokens", "4", "--dtype", "float32", "--block-size", "4", "--block-capacity", "32"])
    assert code == 0
    printed = [int(t) for t in capsys.readouterr().out.strip().splitlines()[-1].split(",")]
    assert printed == pz.greedy_generate(cfg, weights, prompt, 4)


def test_random_weights_model_steps():
    """Seeded random weights for a configuration (what the benchmark uses; the bias table's
    rows come from the configuration then): the model is assembled without a checkpoint and
    its logits do not depend on how the prompt was cut."""
    from forge_engine_b200.engine import ModelRunner

    cfg = pz.written(mixed_config("bfloat16"))
    for layer in cfg["layers"]:
        if layer["type"] == "attention":
            layer["mixer"]["bias_rows"] = 10
    runner = ModelRunner.from_random(cfg, 5, dtype="bfloat16", page_size=16, num_pages=32, max_requests=2, std=0.05)
    tokens = tokens_of(cfg, 40, 3)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 40)]])["a"]
    cut = run_schedule(runner, {"b": tokens}, [[("b", 23)], [("b", 16)], [("b", 1)]])["b"]
    assert torch.isfinite(whole).all()
    assert float((whole - cut).abs().max()) <= 0.05 * max(1.0, float(whole.abs().max()))
