"""A plain, slow restatement of the Nuvivik decoder: whole sequences, no cache, no batch.

One function per mechanism, written from the design's equations with dense tensors and
Python loops (over heads for attention, over tokens for the router).  It shares nothing
with the package: tests compare the engine with it.  ``weights`` maps checkpoint tensor
names to tensors; ``config`` is the dict of config.json.  Everything runs in the dtype of
``work`` (64-bit by default).
"""

from __future__ import annotations

import math

import torch


# -- small pieces ------------------------------------------------------------------------------
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def squared_relu(z):
    return torch.clamp(z, min=0) ** 2


def frequencies(rot: dict) -> list:
    """f_i = base^(-2i / dims) for i < dims / 2, then - if ``scaling`` is given - stretched
    by wavelength: short waves stay, long ones are divided by ``factor``, the ones between
    are blended linearly in original / wavelength."""
    dims, base = rot["dims"], rot["base"]
    out = []
    scaling = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, original = (scaling[k] for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < original / high:
                pass
            elif wave > original / low:
                f = f / factor
            else:
                s = (original / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, n]: the first rot.dims elements of every head are rotated, element i with
    element i + dims / 2, by the angle position * f_i; the rest pass."""
    dims = rot["dims"]
    half = dims // 2
    f = torch.tensor(frequencies(rot), dtype=x.dtype)
    angle = torch.arange(x.shape[0], dtype=x.dtype)[:, None] * f[None, :]         # [T, half]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def windowed_softmax(scores: torch.Tensor, window: int, sink=None) -> torch.Tensor:
    """scores [T, T] (query, key) -> weights: key j is visible to query i when 0 <= i - j <
    window; ``sink`` (a number) joins the denominator as exp(sink), without a key or value."""
    length = scores.shape[0]
    i = torch.arange(length)[:, None]
    j = torch.arange(length)[None, :]
    visible = (i - j >= 0) & (i - j < window)
    masked = scores.masked_fill(~visible, -math.inf)
    top = masked.max(dim=-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, torch.as_tensor(sink, dtype=scores.dtype))
    e = torch.exp(masked - top)
    total = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(torch.as_tensor(sink, dtype=scores.dtype) - top)
    return e / total


# -- mixers ------------------------------------------------------------------------------------
def window_of(m: dict, length: int) -> int:
    """The mixer's window; without a mask every earlier token is visible."""
    return m["mask"]["size"] if m.get("mask") is not None else length


def attention(h, w, prefix, m, eps):
    """Grouped-query attention: biased q/k/v, partial rotation, q and k divided by their root
    mean square after the rotation, capped scores, sliding window, plain softmax."""
    length = h.shape[0]
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[prefix + "q"].T + w[prefix + "q.b"]).view(length, heads, dim)
    k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).view(length, kv_heads, dim)
    v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).view(length, kv_heads, vdim)
    q, k = rms(rotate(q, m["rot"]), eps), rms(rotate(k, m["rot"]), eps)
    out = torch.empty(length, heads, vdim, dtype=h.dtype)
    per = heads // kv_heads
    cap = m.get("softcap")
    for head in range(heads):
        g = head // per
        scores = (q[:, head] @ k[:, g].T) * m["scale"]
        if cap is not None:
            scores = cap * torch.tanh(scores / cap)
        out[:, head] = windowed_softmax(scores, window_of(m, length)) @ v[:, g]
    return out.reshape(length, heads * vdim) @ w[prefix + "o"].T


def latent_attention(h, w, prefix, m, eps):
    """Attention whose keys and values are expanded from one normalised latent per token, with
    one rotated key part shared by the heads, a sliding window and a sink in the softmax."""
    length = h.shape[0]
    heads, dim, rdim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = dict(m["rot"], dims=rdim)
    c_q = rms(h @ w[prefix + "dq"].T, eps) * w[prefix + "dq.norm"]
    q = (c_q @ w[prefix + "uq"].T).view(length, heads, dim + rdim)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], rot)
    down = h @ w[prefix + "dkv"].T
    c = rms(down[:, :rank], eps) * w[prefix + "dkv.norm"]
    k_rot = rotate(down[:, None, rank:], rot)[:, 0]                                 # [T, rdim], one for all heads
    k_plain = (c @ w[prefix + "uk"].T).view(length, heads, dim)
    v = (c @ w[prefix + "uv"].T).view(length, heads, vdim)
    out = torch.empty(length, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        scores = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        out[:, head] = windowed_softmax(scores, window_of(m, length), sink=w[prefix + "sink"][head]) @ v[:, head]
    return out.reshape(length, heads * vdim) @ w[prefix + "o"].T


# -- feed-forwards -----------------------------------------------------------------------------
def dense_feed_forward(h, w, prefix):
    return gelu_tanh(h @ w[prefix + "up"].T) @ w[prefix + "down"].T


def choose(scores: torch.Tensor, top: int, count: int, keep: int) -> list:
    """The experts one token uses.  ``scores`` [experts]; the experts form ``count`` equal
    groups of neighbours, a group is worth the sum of its two largest scores, and only the
    ``keep`` best groups' experts can be chosen; of those, the ``top`` largest scores."""
    experts = scores.shape[0]
    size = experts // count
    worth = []
    for g in range(count):
        members = sorted((float(s) for s in scores[g * size:(g + 1) * size]), reverse=True)
        worth.append(sum(members[:2]))
    open_groups = sorted(range(count), key=lambda g: (-worth[g], g))[:keep]
    allowed = [e for e in range(experts) if e // size in open_groups]
    return sorted(allowed, key=lambda e: (-float(scores[e]), e))[:top]


def routed_feed_forward(h, w, prefix, mlp, chosen_out: list | None = None):
    router = mlp["router"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    scores = torch.sigmoid(h @ w[prefix + "router"].T)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        picked = choose(scores[t], router["top"], groups["count"], groups["keep"])
        if chosen_out is not None:
            chosen_out.append(picked)
        for e in picked:
            unit = f"{prefix}e{e}."
            out[t] += scores[t, e] * (squared_relu(h[t] @ w[unit + "up"].T) @ w[unit + "down"].T)
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
    x = w["embed"][ids] * config["embedding"]["scale"]
    for index, layer in enumerate(config["layers"]):
        pre = f"l{index}."
        if layer["type"] == "attention":
            update = attention(x, w, pre + "mix.", layer["mixer"], eps)
        elif layer["type"] == "latent_attention":
            update = latent_attention(x, w, pre + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms(update, eps) * w[pre + "norm1"]
        if layer.get("mlp") is not None:
            x = x + rms(feed_forward(x, w, pre + "mlp.", layer["mlp"]), eps) * w[pre + "norm2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T * config.get("logit_scale", 1.0)
    cap = config.get("logit_softcap")
    return logits if cap is None else cap * torch.tanh(logits / cap)


# -- tensors, random weights, small configurations ------------------------------------------------
def tensor_shapes(config: dict) -> dict:
    width = config["width"]
    shapes = {"embed": (config["vocab"], width), "final.norm": (width,), "head": (config["vocab"], width)}
    for index, layer in enumerate(config["layers"]):
        pre, m = f"l{index}.", layer["mixer"]
        shapes[pre + "norm1"] = (width,)
        if layer["type"] == "attention":
            q, k, v = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            shapes.update({pre + "mix.q": (q, width), pre + "mix.q.b": (q,), pre + "mix.k": (k, width),
                           pre + "mix.k.b": (k,), pre + "mix.v": (v, width), pre + "mix.v.b": (v,),
                           pre + "mix.o": (width, m["heads"] * m["vdim"])})
        else:
            heads, dim, rdim, vdim = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            shapes.update({pre + "mix.dq": (m["q_rank"], width), pre + "mix.dq.norm": (m["q_rank"],),
                           pre + "mix.uq": (heads * (dim + rdim), m["q_rank"]),
                           pre + "mix.dkv": (m["kv_rank"] + rdim, width), pre + "mix.dkv.norm": (m["kv_rank"],),
                           pre + "mix.uk": (heads * dim, m["kv_rank"]), pre + "mix.uv": (heads * vdim, m["kv_rank"]),
                           pre + "mix.sink": (heads,), pre + "mix.o": (width, heads * vdim)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        shapes[pre + "norm2"] = (width,)
        if mlp.get("kind", "dense") == "dense":
            shapes.update({pre + "mlp.up": (mlp["ff"], width), pre + "mlp.down": (width, mlp["ff"])})
        else:
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                shapes.update({f"{pre}mlp.e{e}.up": (ff, width), f"{pre}mlp.e{e}.down": (width, ff)})
            shapes[pre + "mlp.router"] = (mlp["router"]["experts"], width)
    return shapes


def random_weights(config: dict, seed: int, dtype=torch.bfloat16) -> dict:
    """Seeded weights whose sizes keep activations of order one; stored in ``dtype``."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2") or name == "final.norm":
            t = 0.6 + 0.2 * torch.randn(shape, generator=gen)
        elif last == "norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        elif last == "sink":
            t = torch.randn(shape, generator=gen)
        elif last == "b":
            t = 0.5 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        elif last == "router":
            t = 2.0 * torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        else:
            t = 1.5 * torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


def dense(ff=48):
    return {"kind": "dense", "ff": ff}


def routed(experts=6, top=2, ff=24, groups=(3, 2)):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, window=24, rot_dims=8, base=10000.0, scaling=None, scale=None,
                    softcap=15.0, mlp="dense"):
    """``window`` None leaves the mask out: every earlier token is visible."""
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "rot": rot,
             "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if softcap is not None:
        mixer["softcap"] = softcap
    if window is None:
        del mixer["mask"]
    return {"type": "attention", "mixer": mixer, "mlp": dense() if mlp == "dense" else mlp}


def latent_layer(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=32, kv_rank=40, window=24, base=10000.0, scale=None, mlp="dense"):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim},
             "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if window is None:
        del mixer["mask"]
    return {"type": "latent_attention", "mixer": mixer, "mlp": dense() if mlp == "dense" else mlp}


def config(layers, width=64, vocab=97, eps=1e-5, embedding_scale=0.7, logit_scale=1.5, logit_softcap=25.0) -> dict:
    out = {"architecture": "Nuvivik", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": embedding_scale}, "logit_scale": logit_scale, "layers": list(layers)}
    if logit_softcap is not None:
        out["logit_softcap"] = logit_softcap
    return out


def greedy_generate(cfg: dict, weights: dict, prompt, count: int) -> list:
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(forward(cfg, weights, ids)[-1].argmax()))
    return ids[len(prompt):]
