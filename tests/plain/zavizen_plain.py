"""The Zavizen decoder written out plainly: whole sequences, dense score matrices, Python loops over time, one
function per mechanism.  It shares nothing with the package; the tests run it in float64 on the weights the engine was
given.

    streams  : s copies x_1 .. x_s of the embedding row; a sublayer reads u = sum_s in[s] x_s and writes
               x_t <- sum_s mix[s, t] x_s + out[t] * (scale_vector * sublayer(norm(u)))        all t from the old x
    norm     : u / sqrt(mean(u^2) + eps) * (1 + w)
    a layer  : the mixer sublayer, then the feed-forward sublayer (if the layer has one)
    loop     : the run of layers [start, stop) is walked `times` times (one set of weights, a memory per walk)
    logits   = head(norm(sum_s x_s))

Mixers: ``mamba2`` (a state-space recurrence with a scalar decay per head and token behind a short convolution) and
``parallel`` (softmax attention with queries and keys normed over the whole projection, beside a retention with a
constant decay per head; each side's output normed over the model width, half their sum).  Feed-forwards: dense gated,
or routed experts with softmax scores, groups scored by their best expert, and a shared expert.

``raw`` is the configuration as config.json holds it; ``w`` maps tensor names to tensors.
"""

from __future__ import annotations

import math

import torch

WEIGHT_EPS = 1e-20


def rms_norm(x, weight, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def offset_norm(x, weight, eps):
    """The layers' norm: the stored weight stands around zero."""
    return rms_norm(x, 1.0 + weight, eps)


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(rot):
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = base ** (-2.0 * i / dims)
    scaling = rot.get("scaling")
    if scaling is not None:
        freq = freq / float(scaling["factor"])
    return freq


def rotate_half(x, rot, first=0):
    """x [T, heads, dim]; the first ``dims`` dims of every head turned, dim i with dim i + dims / 2.  The rows stand
    at positions ``first``, ``first + 1``, ..."""
    T = x.shape[0]
    dims = int(rot["dims"])
    freq = rotary_frequencies(rot)
    # positions and angles are float32 in the design: one rounding of the frequency and one of the product
    angle = (torch.arange(first, first + T, dtype=torch.float32)[:, None] * freq.float()[None, :]).double()
    cos, sin = torch.cos(angle).to(x.dtype)[:, None, :], torch.sin(angle).to(x.dtype)[:, None, :]
    out = x.clone()
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    out[..., : dims // 2] = u * cos - v * sin
    out[..., dims // 2: dims] = v * cos + u * sin
    return out


def softmax_attention(h, w, prefix, m, eps):
    """The left side: grouped queries, q and k normed over all their heads at once, partial rotation, causal."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rms_norm(h @ w[f"{prefix}.q"].T, w[f"{prefix}.q.norm"], eps).view(T, H, D)
    k = rms_norm(h @ w[f"{prefix}.k"].T, w[f"{prefix}.k.norm"], eps).view(T, G, D)
    v = (h @ w[f"{prefix}.v"].T).view(T, G, V)
    q, k = rotate_half(q, m["rot"]), rotate_half(k, m["rot"])
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    heads = []
    for i in range(H):
        g = i // (H // G)
        s = (q[:, i] @ k[:, g].T) * float(m["scale"])
        heads.append(torch.softmax(s.masked_fill(~causal, float("-inf")), dim=-1) @ v[:, g])
    return torch.cat(heads, dim=-1) @ w[f"{prefix}.o"].T


def retention(h, w, prefix, m, eps):
    """The right side: S <- decay S + k v^T, o = S^T q per head; no softmax, no denominator."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rotate_half((h @ w[f"{prefix}.q"].T).view(T, H, D), m["rot"])
    k = rotate_half((h @ w[f"{prefix}.k"].T).view(T, H, D), m["rot"]) * D ** -0.5
    v = (h @ w[f"{prefix}.v"].T).view(T, H, V)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(H):
        S = torch.zeros(D, V, dtype=h.dtype)
        for t in range(T):
            S = float(m["decay"][i]) * S + torch.outer(k[t, i], v[t, i])
            out[t, i] = S.T @ q[t, i]
    out = rms_norm(out, None, eps).reshape(T, H * V)
    return (out * silu(h @ w[f"{prefix}.g"].T)) @ w[f"{prefix}.o"].T


def parallel_mixer(h, w, prefix, m, eps):
    left = rms_norm(softmax_attention(h, w, f"{prefix}.left", m["left"], eps), w[f"{prefix}.left.out"], eps)
    right = rms_norm(retention(h, w, f"{prefix}.right", m["right"], eps), w[f"{prefix}.right.out"], eps)
    return 0.5 * (left + right)


def short_convolution(x, weight, bias):
    """x [T, channels]; weight [channels, taps], its last column the current token's; zeros before the start."""
    T, taps = x.shape[0], weight.shape[1]
    padded = torch.cat((torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x), dim=0)
    out = bias.expand(T, -1).clone()
    for j in range(taps):
        out = out + padded[j: j + T] * weight[:, j]
    return out


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def mamba2_mixer(h, w, prefix, m, eps):
    H, P, N, G, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner, T = H * P, h.shape[0]
    p = h @ w[f"{prefix}.in"].T
    z, xbc, dt = p[:, :inner], p[:, inner: 2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, w[f"{prefix}.conv"], w[f"{prefix}.conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner: inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[f"{prefix}.dt_bias"])
    rate = torch.exp(w[f"{prefix}.A_log"])
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for i in range(H):
        g = i // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-rate[i] * dt[t, i]) * S + dt[t, i] * torch.outer(B[t, g], x[t, i])
            y[t, i] = S.T @ C[t, g] + w[f"{prefix}.D"][i] * x[t, i]
    y = y.reshape(T, inner) * silu(z)
    y = rms_norm(y.view(T, parts, inner // parts), None, eps).reshape(T, inner) * w[f"{prefix}.norm"]
    return y @ w[f"{prefix}.o"].T


def gated_expert(h, w, prefix):
    return (silu(h @ w[f"{prefix}.gate"].T) * (h @ w[f"{prefix}.up"].T)) @ w[f"{prefix}.down"].T


def route(logits, router, margins=None):
    """logits [T, experts] -> (chosen [T, top] long, weights [T, top]).  ``margins`` (a list) receives, per token, by
    how much (in logits) the last kept group and the last chosen expert lead the first ones left out."""
    E, top = int(router["experts"]), int(router["top"])
    s = torch.softmax(logits, dim=-1)
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = router.get("groups")
    lead = torch.full((logits.shape[0],), float("inf"), dtype=logits.dtype)
    if groups is not None:
        count, keep = int(groups["count"]), int(groups["keep"])
        best = s.view(-1, count, E // count).max(dim=-1).values
        kept = best.topk(keep, dim=-1).indices
        mask = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        allowed = mask[:, :, None].expand(-1, -1, E // count).reshape(-1, E)
        if keep < count:
            ranked = logits.view(-1, count, E // count).max(dim=-1).values.sort(dim=-1, descending=True).values
            lead = torch.minimum(lead, ranked[:, keep - 1] - ranked[:, keep])
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    if margins is not None:
        ranked = logits.masked_fill(~allowed, float("-inf")).sort(dim=-1, descending=True).values
        if top < int(allowed[0].sum()):
            lead = torch.minimum(lead, ranked[:, top - 1] - ranked[:, top])
        margins.append(lead)
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + WEIGHT_EPS) * float(router["scale"])


def feed_forward(h, w, prefix, mlp, margins=None):
    if mlp.get("kind", "dense") == "dense":
        return gated_expert(h, w, prefix)
    chosen, weights = route(h @ w[f"{prefix}.router"].T, mlp["router"], margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(chosen[t].tolist(), weights[t]):
            out[t] += c * gated_expert(h[t: t + 1], w, f"{prefix}.e{e}")[0]
    if mlp.get("shared") is not None:
        out = out + gated_expert(h, w, f"{prefix}.shared")
    return out


def schedule(raw):
    count = len(raw["layers"])
    loop = raw.get("loop") or {"start": 0, "stop": count, "times": 1}
    order = list(range(loop["start"]))
    for _ in range(int(loop["times"])):
        order += list(range(loop["start"], loop["stop"]))
    return order + list(range(loop["stop"], count))


def sublayer(xs, w, hc, scale_vector, norm_weight, eps, fn):
    """xs [streams, T, width] -> the new streams."""
    u = torch.einsum("s,stw->tw", w[f"{hc}.in"], xs)
    y = fn(offset_norm(u, norm_weight, eps)) * scale_vector
    return torch.einsum("sr,stw->rtw", w[f"{hc}.mix"], xs) + w[f"{hc}.out"][:, None, None] * y


def forward_streams(w, raw, tokens, dtype=torch.float64, margins=None):
    """The sum of the streams after every layer run, [runs, T, width], and the final streams."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(raw["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    xs = x.unsqueeze(0).repeat(int(raw["streams"]), 1, 1)
    after = []
    for i in schedule(raw):
        layer, p = raw["layers"][i], f"l{i}"
        if layer["type"] == "parallel":
            mix = lambda h: parallel_mixer(h, w, f"{p}.mix", layer["mixer"], eps)     # noqa: E731
        else:
            mix = lambda h: mamba2_mixer(h, w, f"{p}.mix", layer["mixer"], eps)       # noqa: E731
        xs = sublayer(xs, w, f"{p}.hc1", w[f"{p}.ls1"], w[f"{p}.norm1"], eps, mix)
        if layer.get("mlp") is not None:
            xs = sublayer(xs, w, f"{p}.hc2", w[f"{p}.ls2"], w[f"{p}.norm2"], eps,
                          lambda h: feed_forward(h, w, f"{p}.mlp", layer["mlp"], margins))
        after.append(xs.sum(0))
    return torch.stack(after), xs


def forward_logits(w, raw, tokens, dtype=torch.float64, margins=None):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    _, xs = forward_streams(w, raw, tokens, dtype, margins)
    return offset_norm(xs.sum(0), w["final.norm"], float(raw["norm"]["eps"])) @ w["head"].T


def forward(raw, w, tokens, margins=None):
    """Logits of every position, [T, vocab], in the dtype of the weights."""
    return forward_logits(w, raw, tokens, dtype=w["embed"].dtype, margins=margins)


def greedy_generate(raw, w, prompt, count):
    ids, out = list(prompt), []
    for _ in range(count):
        token = int(forward(raw, w, ids)[-1].argmax())
        out.append(token)
        ids.append(token)
    return out
