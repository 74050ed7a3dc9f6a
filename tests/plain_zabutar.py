"""A plain, slow restatement of the Zabutar decoder: whole sequences, no cache, no batch.

One function per mechanism, written from the design's equations with dense tensors and
Python loops (over time for the recurrence, over tokens for the router).  It shares nothing
with the package: tests compare the engine with it.  ``weights`` maps checkpoint tensor
names to tensors; ``config`` is the dict of config.json.  Everything runs in the dtype of
``work`` (64-bit by default).
"""

from __future__ import annotations

import math

import torch

RENORM_FLOOR = 1e-20           # added to the sum the chosen experts' scores are divided by


# -- small pieces ------------------------------------------------------------------------------
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, stored, eps):
    """RMS norm whose weight is stored as its distance from one."""
    return rms(x, eps) * (1.0 + stored)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def xielu(z, p, q):
    """Above zero softplus(p) z^2 + z/2; else (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    up = softplus(p) * z * z + 0.5 * z
    neg = torch.clamp(z, max=0)
    down = (0.5 + softplus(q)) * (torch.expm1(neg) - neg) + 0.5 * neg
    return torch.where(z > 0, up, down)


def short_convolution(h, taps_weight):
    """h [T, C] -> h + conv(h): channel by channel, out_t += sum_j w[:, j] h_(t - taps + 1 + j),
    with zeros before the first token."""
    length, taps = h.shape[0], taps_weight.shape[1]
    out = h.clone()
    for j in range(taps):
        back = taps - 1 - j
        if back < length:
            out[back:] += taps_weight[:, j] * h[: length - back]
    return out


# -- mixers ------------------------------------------------------------------------------------
def gated_recurrence(h, w, prefix, m, eps):
    """The mixer "hgrn2": per head a state [dim, vdim]; the forget gate f (bounded below by a
    learned value) scales the state's rows, and 1 - f is what writes the value into them."""
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    length = h.shape[0]
    q = torch.nn.functional.silu(h @ w[prefix + "q"].T).view(length, heads, dim)
    v = (h @ w[prefix + "v"].T).view(length, heads, vdim)
    low = w[prefix + "lower"].view(heads, dim)
    f = low + (1.0 - low) * torch.sigmoid(h @ w[prefix + "f"].T + w[prefix + "f.b"]).view(length, heads, dim)
    state = torch.zeros(heads, dim, vdim, dtype=h.dtype)
    out = torch.empty(length, heads, vdim, dtype=h.dtype)
    for t in range(length):
        state = f[t][:, :, None] * state + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    out = rms(out, eps) * w[prefix + "norm"]
    return out.reshape(length, heads * vdim) @ w[prefix + "o"].T


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the bias table for a distance n >= 0: one row per distance below rows/2, then
    rows that widen logarithmically until ``far``, where the last row takes over."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def biased_attention(h, w, prefix, m, kv_prefix=None):
    """The mixer "attention": grouped-query softmax attention without rotation; a learned
    table adds a bias by (bucketed) distance and head.  ``kv_prefix``: the layer whose keys
    and values are used (its projections applied to ITS input happen elsewhere; here the
    caller hands k and v through ``m['_kv']`` when they come from another layer)."""
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    length = h.shape[0]
    q = (h @ w[prefix + "q"].T).view(length, heads, dim)
    if m.get("_kv") is not None:
        k, v = m["_kv"]
    else:
        k = (h @ w[prefix + "k"].T).view(length, kv_heads, dim)
        v = (h @ w[prefix + "v"].T).view(length, kv_heads, vdim)
    table = w[prefix + "rel"].to(h.dtype)
    rows = table.shape[0]
    buckets = torch.tensor([[distance_bucket(i - j, rows, m["bias_max"]) if j <= i else 0 for j in range(length)]
                            for i in range(length)])
    causal = torch.arange(length)[None, :] <= torch.arange(length)[:, None]
    out = torch.empty(length, heads, vdim, dtype=h.dtype)
    per = heads // kv_heads
    for head in range(heads):
        g = head // per
        scores = (q[:, head] @ k[:, g].T) * m["scale"] + table[:, head][buckets]
        scores = scores.masked_fill(~causal, float("-inf"))
        out[:, head] = torch.softmax(scores, dim=-1) @ v[:, g]
    return out.reshape(length, heads * vdim) @ w[prefix + "o"].T, (k, v)


# -- feed-forwards -----------------------------------------------------------------------------
def dense_feed_forward(h, w, prefix):
    p, q = w[prefix + "act"][0], w[prefix + "act"][1]
    z = h @ w[prefix + "up"].T + w[prefix + "up.b"]
    return xielu(z, p, q) @ w[prefix + "down"].T + w[prefix + "down.b"]


def gated_unit(h, w, prefix):
    return (torch.nn.functional.silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(logits, correction, top, groups, keep, scale):
    """logits [E] of one token -> list of (expert, weight).  Choice by score + correction among
    the experts of the ``keep`` best groups (a group's mark is its largest choice score);
    weights from the scores alone, divided by their sum, times ``scale``."""
    scores = torch.softmax(logits, dim=-1)
    choice = scores + correction
    count = logits.shape[0]
    size = count // groups
    marks = [max(float(c) for c in choice[g * size : (g + 1) * size]) for g in range(groups)]
    # ties: the lower index wins, for groups and for experts
    best = sorted(range(groups), key=lambda g: (-marks[g], g))[:keep]
    allowed = [e for e in range(count) if e // size in best]
    chosen = sorted(allowed, key=lambda e: (-float(choice[e]), e))[:top]
    total = sum(scores[e] for e in chosen) + RENORM_FLOOR
    return [(e, scores[e] / total * scale) for e in chosen]


def routed_feed_forward(h, w, prefix, mlp):
    r = mlp["router"]
    real, identity = r["experts"], r.get("identity", 0)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    logits = h @ w[prefix + "router"].T
    correction = w[prefix + "correction"].to(h.dtype)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for expert, weight in route(logits[t], correction, r["top"], groups["count"], groups["keep"], r["scale"]):
            if expert >= real:
                out[t] += weight * h[t]          # an identity expert hands its input on
            else:
                out[t] += weight * gated_unit(h[t : t + 1], w, f"{prefix}e{expert}.")[0]
    if mlp.get("shared") is not None:
        out = out + gated_unit(h, w, prefix + "shared.")
    return out


def feed_forward(h, w, prefix, mlp):
    if mlp.get("kind", "dense") == "dense":
        return dense_feed_forward(h, w, prefix)
    return routed_feed_forward(h, w, prefix, mlp)


# -- the model ---------------------------------------------------------------------------------
def forward(config: dict, weights: dict, tokens, work=torch.float64, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  ``layers_out`` collects the residual stream after every layer."""
    w = {k: (v.to(work) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][ids] + w["pos"][: len(ids)]
    kept: dict = {}                                   # layer -> (k, v) of attention layers
    for index, layer in enumerate(config["layers"]):
        pre = f"l{index}."
        m = dict(layer["mixer"])
        h = short_convolution(offset_norm(x, w[pre + "norm1"], eps), w[pre + "canon1"])
        if layer["type"] == "hgrn2":
            update = gated_recurrence(h, w, pre + "mix.", m, eps)
        elif layer["type"] == "attention":
            m["_kv"] = kept[m["kv_from"]] if m.get("kv_from") is not None else None
            update, kept[index] = biased_attention(h, w, pre + "mix.", m)
        else:
            raise ValueError(layer["type"])
        x = x + offset_norm(update, w[pre + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = short_convolution(offset_norm(x, w[pre + "norm2"], eps), w[pre + "canon2"])
            x = x + offset_norm(feed_forward(h, w, pre + "mlp.", layer["mlp"]), w[pre + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T


# -- tensors, random weights, small configurations ------------------------------------------------
def tensor_shapes(config: dict) -> dict:
    width, taps = config["width"], config["canon"]["taps"]
    shapes = {"embed": (config["vocab"], width), "pos": (config["max_positions"], width),
              "final.norm": (width,), "head": (config["vocab"], width)}
    for index, layer in enumerate(config["layers"]):
        pre, m = f"l{index}.", layer["mixer"]
        for name in ("norm1", "norm1b"):
            shapes[pre + name] = (width,)
        shapes[pre + "canon1"] = (width, taps)
        if layer["type"] == "hgrn2":
            qk, v = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            shapes.update({pre + "mix.q": (qk, width), pre + "mix.f": (qk, width), pre + "mix.f.b": (qk,),
                           pre + "mix.lower": (qk,), pre + "mix.v": (v, width), pre + "mix.norm": (m["vdim"],),
                           pre + "mix.o": (width, v)})
        else:
            shapes[pre + "mix.q"] = (m["heads"] * m["dim"], width)
            if m.get("kv_from") is None:
                shapes[pre + "mix.k"] = (m["kv_heads"] * m["dim"], width)
                shapes[pre + "mix.v"] = (m["kv_heads"] * m["vdim"], width)
            shapes[pre + "mix.rel"] = (m.get("_bias_rows", 12), m["heads"])
            shapes[pre + "mix.o"] = (width, m["heads"] * m["vdim"])
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        for name in ("norm2", "norm2b"):
            shapes[pre + name] = (width,)
        shapes[pre + "canon2"] = (width, taps)
        if mlp.get("kind", "dense") == "dense":
            shapes.update({pre + "mlp.up": (mlp["ff"], width), pre + "mlp.up.b": (mlp["ff"],),
                           pre + "mlp.down": (width, mlp["ff"]), pre + "mlp.down.b": (width,), pre + "mlp.act": (2,)})
        else:
            r = mlp["router"]
            for e in range(r["experts"]):
                ff = mlp["expert"]["ff"]
                shapes.update({f"{pre}mlp.e{e}.gate": (ff, width), f"{pre}mlp.e{e}.up": (ff, width),
                               f"{pre}mlp.e{e}.down": (width, ff)})
            outputs = r["experts"] + r.get("identity", 0)
            shapes[pre + "mlp.router"] = (outputs, width)
            shapes[pre + "mlp.correction"] = (outputs,)
            if mlp.get("shared") is not None:
                ff = mlp["shared"]["ff"]
                shapes.update({pre + "mlp.shared.gate": (ff, width), pre + "mlp.shared.up": (ff, width),
                               pre + "mlp.shared.down": (width, ff)})
    return shapes


def random_weights(config: dict, seed: int, dtype=torch.bfloat16) -> dict:
    """Seeded weights whose sizes keep activations of order one; stored in ``dtype``."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            t = 0.2 * torch.randn(shape, generator=gen)                  # stored around zero
        elif name.endswith("mix.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        elif last in ("canon1", "canon2"):
            t = 0.4 * torch.randn(shape, generator=gen)
        elif name.endswith("mix.lower"):
            t = torch.rand(shape, generator=gen) * 0.9
        elif name.endswith("mix.rel"):
            t = 1.5 * torch.randn(shape, generator=gen)
        elif name.endswith("mlp.act"):
            t = torch.randn(shape, generator=gen)
        elif name.endswith("correction"):
            t = 0.1 * torch.randn(shape, generator=gen)
        elif name.endswith(".b"):
            t = 0.5 * torch.randn(shape, generator=gen)
        elif name in ("embed", "pos"):
            t = torch.randn(shape, generator=gen)
        elif name.endswith("router"):
            t = 2.0 * torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        else:
            t = 1.5 * torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


def dense(ff=48):
    return {"kind": "dense", "ff": ff}


def routed(experts=5, identity=1, top=2, ff=24, groups=(3, 2), scale=1.5, shared_ff=40):
    mlp = {"kind": "moe", "expert": {"ff": ff},
           "router": {"experts": experts, "identity": identity, "top": top, "scale": scale,
                      "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared_ff is not None:
        mlp["shared"] = {"ff": shared_ff}
    return mlp


def recurrent_layer(heads=4, dim=8, vdim=16, mlp="dense"):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": dense() if mlp == "dense" else mlp}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, scale=None, bias_rows=12, bias_max=40, kv_from=None, mlp="dense"):
    # "_bias_rows" is not a key of config.json (the table's shape says it): ``written`` drops it
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "_bias_rows": bias_rows, "bias_max": bias_max,
             "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": dense() if mlp == "dense" else mlp}


def config(layers, width=64, vocab=97, eps=1e-5, taps=3, max_positions=512) -> dict:
    return {"architecture": "Zabutar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps},
            "max_positions": max_positions, "layers": list(layers)}


def written(cfg: dict) -> dict:
    """The configuration as config.json holds it: without the keys that only size random tensors."""
    def strip(item):
        if isinstance(item, dict):
            return {k: strip(v) for k, v in item.items() if not k.startswith("_")}
        if isinstance(item, list):
            return [strip(v) for v in item]
        return item
    return strip(cfg)


def greedy_generate(cfg: dict, weights: dict, prompt, count: int) -> list:
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(forward(cfg, weights, ids)[-1].argmax()))
    return ids[len(prompt):]
