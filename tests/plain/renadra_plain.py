"""The Renadra decoder written out plainly: whole sequences, dense score matrices, Python loops over time, one
function per mechanism.  It shares nothing with the package; the tests run it in float64 (or float32) on the weights
the engine was given.

    x_0      = embed[token] * scale + bigram[(prev * mul_prev + token * mul_cur) mod buckets]   (row `buckets` at t = 0)
    a pass   : x <- x + mixer(norm_1(x));  x <- x + ff(norm_2(x))   for the layers of the pass
    loop     : the run of layers [start, stop) is walked `times` times (one set of weights, a memory per walk); x_0 is added to x before
               every pass but the first
    logits   = head(norm(x))

Mixers: ``attention`` (rotated queries and keys in neighbouring pairs, unit-RMS values, a window, softmax),
``hgrn2`` (a matrix memory per head that writes to a row with one minus its forget gate), ``parallel`` (attention without
a softmax, whose values are its unrotated keys, beside a linear attention with a constant decay per head).

``raw`` is the configuration as config.json holds it; ``w`` maps tensor names to tensors.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z):
    return z * torch.sigmoid(z)


def embed(tokens, w, raw):
    """Scaled rows plus the row of the (previous token, token) pair's bucket; the first token takes the last row."""
    e = raw["embedding"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][ids] * float(e["scale"])
    b = e.get("bigram")
    if b is not None:
        rows = torch.empty_like(ids)
        rows[0] = b["buckets"]
        rows[1:] = (ids[:-1] * b["mul_prev"] + ids[1:] * b["mul_cur"]) % b["buckets"]
        x = x + w["bigram"][rows]
    return x


def rotary_frequencies(rot):
    """(frequency per pair [dims / 2] in float64, factor on cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    s = rot.get("scaling")
    if s is None:
        return freq, 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(s["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(s["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, rot, layout):
    """x [T, heads, dim]; the first ``dims`` dims of every head turned by the position's angles.  ``layout``:
    ``"half"`` pairs dim i with i + dims / 2, ``"pairs"`` dim 2i with 2i + 1."""
    T = x.shape[0]
    dims = int(rot["dims"])
    freq, factor = rotary_frequencies(rot)
    # the design forms positions and angles in float32: one rounding of the frequency and one of the product
    angle = (torch.arange(T, dtype=torch.float32)[:, None] * freq.float()[None, :]).double()
    cos = (torch.cos(angle) * factor).to(x.dtype)[:, None, :]
    sin = (torch.sin(angle) * factor).to(x.dtype)[:, None, :]
    out = x.clone()
    if layout == "half":
        u, v = x[..., : dims // 2], x[..., dims // 2: dims]
        out[..., : dims // 2] = u * cos - v * sin
        out[..., dims // 2: dims] = v * cos + u * sin
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    return out


def visible(T, size, keep_first=0):
    """[T, T] bool: i sees j <= i with i - j < size, or j < keep_first."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def linear(h, w, name):
    y = h @ w[name].T
    return y + w[name + ".b"] if name + ".b" in w else y


def attention_mixer(h, w, prefix, m, eps):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rotate(linear(h, w, f"{prefix}.q").view(T, H, D), m["rot"], "pairs")
    k = rotate(linear(h, w, f"{prefix}.k").view(T, G, D), m["rot"], "pairs")
    v = rms_norm(linear(h, w, f"{prefix}.v").view(T, G, V), None, eps)
    see = visible(T, m["mask"]["size"])
    heads = []
    for i in range(H):
        g = i // (H // G)
        s = (q[:, i] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~see, float("-inf"))
        heads.append(torch.softmax(s, dim=-1) @ v[:, g])
    return linear(torch.cat(heads, dim=-1), w, f"{prefix}.o")


def sigmoid_attention(h, w, prefix, m):
    """The left half of ``parallel``: values are the keys before their rotation, capped scores, a window that also
    keeps the first tokens, and a sigmoid in place of the softmax."""
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = linear(h, w, f"{prefix}.q").view(T, H, D)
    k = linear(h, w, f"{prefix}.k").view(T, G, D)
    v = k
    q, k = rotate(q, m["rot"], "half"), rotate(k, m["rot"], "half")
    see = visible(T, m["mask"]["size"], m["mask"].get("keep_first", 0))
    cap = float(m["softcap"])
    heads = []
    for i in range(H):
        g = i // (H // G)
        s = (q[:, i] @ k[:, g].T) * float(m["scale"])
        s = cap * torch.tanh(s / cap)
        p = torch.sigmoid(s + w[f"{prefix}.pb"][i]) * see
        heads.append(p @ v[:, g])
    return torch.cat(heads, dim=-1) @ w[f"{prefix}.o"].T


def decayed_memory(q, k, v, decay):
    """One head.  q [T, D]; k, decay [T, D] (what is written to, and what stays of, each row); v [T, V].
    S_t = diag(decay_t) S_(t-1) + k_t v_t^T from S = 0; o_t = S_t^T q_t."""
    T, D = q.shape
    S = q.new_zeros(D, v.shape[1])
    out = []
    for t in range(T):
        S = decay[t][:, None] * S + torch.outer(k[t], v[t])
        out.append(S.T @ q[t])
    return torch.stack(out)


def lightning_mixer(h, w, prefix, m, eps):
    """The right half of ``parallel``."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ w[f"{prefix}.q"].T).view(T, H, D)
    k = silu(h @ w[f"{prefix}.k"].T).view(T, H, D)
    v = silu(h @ w[f"{prefix}.v"].T).view(T, H, V)
    heads = [decayed_memory(q[:, i], k[:, i], v[:, i], q.new_full((T, D), float(m["decay"][i]))) for i in range(H)]
    o = rms_norm(torch.cat(heads, dim=-1), w[f"{prefix}.norm"], eps)
    return (o * torch.sigmoid(h @ w[f"{prefix}.g"].T)) @ w[f"{prefix}.o"].T


def parallel_mixer(h, w, prefix, m, eps):
    left = sigmoid_attention(h, w, f"{prefix}.left", m["left"])
    right = lightning_mixer(h, w, f"{prefix}.right", m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def hgrn2_mixer(h, w, prefix, m, eps):
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ w[f"{prefix}.q"].T).view(T, H, D)
    v = (h @ w[f"{prefix}.v"].T).view(T, H, V)
    low = w[f"{prefix}.lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w[f"{prefix}.f"].T + w[f"{prefix}.f.b"])).view(T, H, D)
    heads = [rms_norm(decayed_memory(q[:, i], 1.0 - f[:, i], v[:, i], f[:, i]), w[f"{prefix}.norm"], eps)
             for i in range(H)]
    return torch.cat(heads, dim=-1) @ w[f"{prefix}.o"].T


def dense_ff(h, w, prefix):
    return (silu(h @ w[f"{prefix}.gate"].T) * (h @ w[f"{prefix}.up"].T)) @ w[f"{prefix}.down"].T


def layer_order(raw):
    """[(layer, starts a pass after the first)] in the order the layers run."""
    n = len(raw["layers"])
    loop = raw.get("loop")
    if not loop or int(loop["times"]) <= 1:
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(start)]
    for p in range(times):
        order += [(i, p > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(raw, w, tokens, return_layers=False):
    eps = float(raw["norm"]["eps"])
    x0 = embed(tokens, w, raw)
    x = x0
    layers = []
    for i, again in layer_order(raw):
        layer = raw["layers"][i]
        if again:
            x = x + x0
        h = rms_norm(x, w[f"l{i}.norm1"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            y = attention_mixer(h, w, f"l{i}.mix", m, eps)
        elif kind == "hgrn2":
            y = hgrn2_mixer(h, w, f"l{i}.mix", m, eps)
        elif kind == "parallel":
            y = parallel_mixer(h, w, f"l{i}.mix", m, eps)
        else:
            raise ValueError(f"unknown mixer {kind!r}")
        x = x + y
        if layer.get("mlp") is not None:
            x = x + dense_ff(rms_norm(x, w[f"l{i}.norm2"], eps), w, f"l{i}.mlp")
        layers.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits


def greedy_generate(raw, w, prompt, new_tokens):
    tokens = list(prompt)
    for _ in range(new_tokens):
        tokens.append(int(forward(raw, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
