"""The kernels of the Renadra mixers, each alone, against the plain implementation's functions (float64), in float32
and bfloat16 storage: the rotation of queries and keys in both layouts with the value's preparation and the cache
write; attention whose window keeps the first keys and whose weights are sigmoids (prompt tiles and single decoded
tokens, one split and several, inputs built so that one key far back, a key just inside or just outside the window
or the kept keys decides the result); the linear-memory scan in both modes (whole, in portions, token by token,
through state slots that are used again, a value written hundreds of tokens back); the norm of what it reads out; the
pair table's rows with the previous token kept across steps; the two small kernels on the stream."""

import math

import pytest
import torch

from plain import renadra_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: dict(atol=2e-5, rtol=2e-5), torch.bfloat16: dict(atol=2e-2, rtol=2e-2)}


def _ops():
    from ampere_kv_engine_b200.kernels import ops
    return ops


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


# ----------------------------------------------------------------------------- rotation, value, cache write

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot_dims,layout,scaling,from_key,vnorm", [
    (4, 2, 24, 24, 16, "half", (4.0, 32, 8.0, 2.0), True, False),
    (6, 3, 16, 8, 16, "pairs", None, False, True),
    (1, 1, 32, 40, 8, "pairs", None, False, False),
    (8, 2, 64, 64, 64, "half", (8.0, 128, 32.0, 1.0), True, False),
    (3, 3, 20, 12, 4, "half", None, False, True)])
def test_rotary_prep(dtype, heads, kv_heads, dim, vdim, rot_dims, layout, scaling, from_key, vnorm):
    ops = _ops()
    from ampere_kv_engine_b200.config.spec import PartSpec
    from ampere_kv_engine_b200.parts.base import POSITION_ENCODINGS, build_part
    n, page_size, pages, eps = 41, 8, 9, 1e-5
    rot = {"dims": rot_dims, "base": 500.0}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    rope = build_part(POSITION_ENCODINGS, PartSpec("rope", {"theta": rot["base"], "rotary_dim": rot_dims,
                                                           "layout": layout, "scaling": rot.get("scaling")}),
                      hidden_size=8, dtype=dtype, device=torch.device("cuda"))
    freq, dims, lay, factor = rope.rotary_table()
    want_freq, want_factor = plain.rotary_frequencies(rot)
    torch.testing.assert_close(freq.double().cpu(), want_freq, atol=0, rtol=1e-7)
    assert factor == pytest.approx(want_factor) and dims == rot_dims and lay == layout
    g = torch.Generator(device="cuda").manual_seed(5)
    width = (heads + kv_heads) * dim + (0 if from_key else kv_heads * vdim)
    x = (3.0 * torch.randn((n, width), generator=g, device="cuda")).to(dtype)
    positions = torch.randint(0, 3000, (n,), generator=g, device="cuda").to(torch.int32)
    positions[0] = 0
    slots = torch.randperm(pages * page_size, generator=g, device="cuda")[:n].to(torch.int32)
    slots[5] = -1
    k_cache = torch.zeros((pages, kv_heads, page_size, dim), device="cuda", dtype=dtype)
    v_cache = torch.zeros((pages, kv_heads, page_size, vdim), device="cuda", dtype=dtype)
    q = ops.rotary_prep(x, positions, slots, freq, k_cache, v_cache, num_heads=heads, num_kv_heads=kv_heads,
                        head_dim=dim, v_dim=vdim, rotary_dims=dims, layout=lay, factor=factor, value_from_key=from_key,
                        value_norm=vnorm, eps=eps)
    xd = x.double().cpu()
    a, b = heads * dim, kv_heads * dim

    def turned(t):          # the plain rotation works on positions 0 .. T - 1: turn every row at its own position
        rows = []
        for i in range(n):
            p = int(positions[i])
            padded = torch.zeros(p + 1, t.shape[1], t.shape[2], dtype=torch.float64)
            padded[p] = t[i]
            rows.append(plain.rotate(padded, rot, layout)[p])
        return torch.stack(rows)

    kd = xd[:, a:a + b].view(n, kv_heads, dim)
    torch.testing.assert_close(q.double().cpu().view(n, heads, dim), turned(xd[:, :a].view(n, heads, dim)), **TOL[dtype])
    if from_key:
        want_v = kd
    else:
        want_v = xd[:, a + b:].view(n, kv_heads, vdim)
        if vnorm:
            want_v = plain.rms_norm(want_v, None, eps)
    want_k = turned(kd)
    for i in range(n):
        s = int(slots[i])
        if s < 0:
            continue
        torch.testing.assert_close(k_cache[s // page_size, :, s % page_size].double().cpu(), want_k[i], **TOL[dtype])
        torch.testing.assert_close(v_cache[s // page_size, :, s % page_size].double().cpu(), want_v[i], **TOL[dtype])
    written = {int(s) for s in slots.tolist() if s >= 0}
    untouched = [s for s in range(pages * page_size) if s not in written]
    assert float(k_cache.view(pages, kv_heads, page_size, dim)[[s // page_size for s in untouched], :,
                                                              [s % page_size for s in untouched]].abs().sum()) == 0.0


# ----------------------------------------------------------------------------- attention: kept first keys, sigmoids

class _Case:
    """Requests over a shuffled page pool; pages that a window has given back hold NaN and are absent from the table."""

    def __init__(self, dtype, heads, kv_heads, dim, vdim, page, q_lens, ctx_lens, window, keep, seed=0, q_tile=8):
        g = torch.Generator().manual_seed(seed)
        self.dtype, self.heads, self.kv_heads, self.dim, self.vdim, self.page = dtype, heads, kv_heads, dim, vdim, page
        self.q_lens, self.ctx_lens, self.window, self.keep = q_lens, ctx_lens, window, keep
        self.k = [torch.randn(c, kv_heads, dim, generator=g).to(dtype) for c in ctx_lens]
        self.v = [torch.randn(c, kv_heads, vdim, generator=g).to(dtype) for c in ctx_lens]
        self.q = [torch.randn(n, heads, dim, generator=g).to(dtype) for n in q_lens]
        self.order = torch.randperm(sum((c + page - 1) // page for c in ctx_lens) + 5, generator=g).tolist()
        cu = [0]
        for n in q_lens:
            cu.append(cu[-1] + n)
        self.cu = cu
        rows = 1 if max(q_lens) == 1 else q_tile
        tiles = [(s, cu[s] + q0, min(rows, n - q0)) for s, n in enumerate(q_lens) for q0 in range(0, n, rows)]
        self.rows, self.tiles = rows, [_i32([t[i] for t in tiles]) for i in range(3)]

    def caches(self):
        pool, page = len(self.order), self.page
        k_cache = torch.full((pool, self.kv_heads, page, self.dim), float("nan")).to(self.dtype)
        v_cache = torch.full((pool, self.kv_heads, page, self.vdim), float("nan")).to(self.dtype)
        table = torch.full((len(self.ctx_lens), max((c + page - 1) // page for c in self.ctx_lens)), -1, dtype=torch.int32)
        order = list(self.order)
        for s, (n, c) in enumerate(zip(self.q_lens, self.ctx_lens)):
            first_query = c - n
            needed = set(range(min(self.keep, c))) | set(range(max(0, first_query - self.window + 1) if self.window else 0, c))
            for lp in sorted({key // page for key in needed}):
                pp = order.pop()
                table[s, lp] = pp
                lo, hi = lp * page, min(c, (lp + 1) * page)
                k_cache[pp, :, :hi - lo] = self.k[s][lo:hi].transpose(0, 1)
                v_cache[pp, :, :hi - lo] = self.v[s][lo:hi].transpose(0, 1)
        return k_cache.cuda(), v_cache.cuda(), table.cuda()

    def run(self, ops, *, scale, softcap, sigmoid, bias, splits, out_scale=1.0, kernel="auto"):
        k_cache, v_cache, table = self.caches()
        q = torch.cat([x.reshape(x.shape[0], -1) for x in self.q]).cuda()
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = ops.scored_attention(
            q, k_cache, v_cache, table, _i32(self.cu), _i32(self.ctx_lens), *self.tiles, num_tiles=len(self.tiles[0]),
            q_tile=self.rows, num_splits=splits, num_heads=self.heads, num_kv_heads=self.kv_heads, v_dim=self.vdim,
            scale=scale, window=self.window, softcap=softcap, keep_first=self.keep, sigmoid_weights=sigmoid,
            head_bias=None if bias is None else bias.cuda(), out_scale=out_scale, status=status, kernel=kernel)
        assert int(status.item()) == 0
        return out.double().cpu()

    def reference(self, *, scale, softcap, sigmoid, bias, out_scale=1.0):
        outs = []
        group = self.heads // self.kv_heads
        for s, (n, c) in enumerate(zip(self.q_lens, self.ctx_lens)):
            see = plain.visible(c, self.window or c, self.keep)[c - n:]
            k, v, q = self.k[s].double(), self.v[s].double(), self.q[s].double()
            heads = []
            for h in range(self.heads):
                sc = (q[:, h] @ k[:, h // group].T) * scale
                if softcap:
                    sc = softcap * torch.tanh(sc / softcap)
                if sigmoid:
                    p = torch.sigmoid(sc + (0.0 if bias is None else bias[h].double())) * see
                else:
                    p = torch.softmax(sc.masked_fill(~see, float("-inf")), -1)
                heads.append(p @ v[:, h // group] * out_scale)
            outs.append(torch.cat(heads, dim=-1))
        return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sigmoid", [True, False])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,page,window,keep", [(4, 2, 24, 24, 16, 13, 5), (3, 3, 16, 8, 8, 40, 0),
                                                                       (8, 2, 64, 64, 16, 33, 17), (2, 1, 20, 36, 4, 9, 9)])
def test_attention_with_kept_first_keys_prompts_and_decoded_tokens(dtype, sigmoid, heads, kv_heads, dim, vdim, page,
                                                                   window, keep):
    ops = _ops()
    bias = torch.linspace(-2.0, 0.5, heads) if sigmoid else None
    kw = dict(scale=1.7 * dim ** -0.5, softcap=6.0 if sigmoid else 0.0, sigmoid=sigmoid, bias=bias)
    # prompt portions: from the first token, behind a long context, a portion of two tokens, one of one token
    case = _Case(dtype, heads, kv_heads, dim, vdim, page, [47, 30, 2, 1, 70], [47, 230, 95, 1, 71], window, keep, seed=3)
    for splits in (1, 3):
        torch.testing.assert_close(case.run(ops, splits=splits, **kw), case.reference(**kw), **TOL[dtype])
    # decoded tokens: contexts around the window's and the kept keys' sizes and around page borders
    ctx = [1, 2, keep + 1, keep + 2, window - 1, window, window + 1, window + keep, window + keep + 1, 2 * page, 2 * page + 1,
           300, 301]
    ctx = [c for c in ctx if c >= 1]
    case = _Case(dtype, heads, kv_heads, dim, vdim, page, [1] * len(ctx), ctx, window, keep, seed=4)
    for splits in (1, 2, 5):
        torch.testing.assert_close(case.run(ops, splits=splits, out_scale=0.8, **kw), case.reference(out_scale=0.8, **kw),
                                   **TOL[dtype])


@pytest.mark.parametrize("sigmoid", [True, False])
@pytest.mark.parametrize("heads,kv_heads,page,window,keep", [(8, 2, 16, 200, 70), (4, 4, 64, 130, 64), (16, 2, 32, 257, 1),
                                                             (8, 1, 128, 96, 130), (8, 2, 16, 300, 0)])
def test_prompt_tiles_of_128_dims_on_the_tensor_cores(sigmoid, heads, kv_heads, page, window, keep):
    """bfloat16 heads of 128 dims take the tcgen05 prompt kernel: kept keys whose count is no multiple of a block or a
    box, windows that start right behind them, among them and far from them, pages between the two that were given
    back, portions of two tokens and of one, against the plain attention and against the general kernel."""
    ops = _ops()
    dtype, dim = torch.bfloat16, 128
    assert ops.scored_takes_tensor_cores(dtype, dim, dim, heads // kv_heads, page, prompt=True)
    q_tile = ops.attention_q_tile(dim, heads // kv_heads)
    bias = torch.linspace(-3.0, -1.0, heads) if sigmoid else None
    kw = dict(scale=1.3 * dim ** -0.5, softcap=8.0, sigmoid=sigmoid, bias=bias, out_scale=0.7)
    q_lens = [150, 40, 2, 1, 333, 64]
    ctx_lens = [150, 700, keep + window + 9, 1, 333 + window + keep + 61, max(64, keep + 70)]
    case = _Case(dtype, heads, kv_heads, dim, dim, page, q_lens, ctx_lens, window, keep, seed=21, q_tile=q_tile)
    got = case.run(ops, splits=1, **kw)
    want = case.reference(**kw)
    assert bool(torch.isfinite(got).all())
    # weights rounded to bfloat16 before they meet the values: a few parts in a thousand of a row's scale
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-3)
    assert float(((got - want).abs() / scale).max()) < 2.5e-2
    general = case.run(ops, splits=1, kernel="general", **kw)
    assert float(((got - general).abs() / scale).max()) < 2.5e-2


@pytest.mark.parametrize("sigmoid", [True, False])
@pytest.mark.parametrize("heads,kv_heads,dim,page,window,keep", [(8, 2, 128, 16, 200, 70), (4, 4, 64, 64, 130, 64),
                                                                 (16, 2, 128, 32, 257, 1), (8, 1, 64, 8, 96, 130),
                                                                 (8, 2, 128, 16, 300, 0)])
def test_decoded_tokens_of_64_and_128_dims_on_the_tensor_cores(sigmoid, heads, kv_heads, dim, page, window, keep):
    """Single tokens of bfloat16 heads take the TMA + mma.sync kernel with 1, 2, 4 or 8 key splits: contexts around the
    kept keys' and the window's sizes, around blocks of 32 keys and page borders, windows that start right behind the
    kept keys, among them and far from them (the pages between were given back), against the plain attention and
    against the general kernel."""
    ops = _ops()
    dtype = torch.bfloat16
    assert ops.scored_takes_tensor_cores(dtype, dim, dim, heads // kv_heads, page, prompt=False)
    bias = torch.linspace(-3.0, -1.0, heads) if sigmoid else None
    kw = dict(scale=1.3 * dim ** -0.5, softcap=8.0, sigmoid=sigmoid, bias=bias, out_scale=0.7)
    edge = (keep + 31) // 32 * 32
    ctx = [1, 2, 31, 32, 33, keep, keep + 1, keep + 2, window - 1, window, window + 1, window + keep, window + keep + 1,
           window + edge, window + edge + 1, window + edge + page, window + edge + page + 1, 2 * page, 2 * page + 1, 700,
           1501]
    ctx = [c for c in ctx if c >= 1]
    case = _Case(dtype, heads, kv_heads, dim, dim, page, [1] * len(ctx), ctx, window, keep, seed=23)
    want = case.reference(**kw)
    scale = want.abs().amax(dim=-1, keepdim=True).clamp_min(1e-3)
    general = case.run(ops, splits=1, kernel="general", **kw)
    assert float(((general - want).abs() / scale).max()) < 2.5e-2
    for splits in (1, 2, 4, 8):
        got = case.run(ops, splits=splits, **kw)
        assert bool(torch.isfinite(got).all())
        # weights rounded to bfloat16 before they meet the values: a few parts in a thousand of a row's scale
        assert float(((got - want).abs() / scale).max()) < 2.5e-2, splits
        assert float(((got - general).abs() / scale).max()) < 2.5e-2, splits


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_key_decides_inside_and_outside_the_window_and_the_kept_keys(dtype):
    """All values are zero but one key's, whose score is made large: the output is that value where the key is
    visible (the last key of the window, the last kept key, a kept key hundreds of positions back) and zero where it
    is just outside, in prompts and in decoding."""
    ops = _ops()
    heads, kv_heads, dim, vdim, page, window, keep, c = 2, 1, 16, 16, 8, 11, 6, 400
    bias = torch.tensor([-30.0, -30.0])                  # a key with an ordinary score weighs about nothing
    kw = dict(scale=1.0, softcap=100.0, sigmoid=True, bias=bias)
    for q_lens in ([1], [37]):
        for marked, seen_by_last in ((c - window, True), (c - window - 1, False), (keep - 1, True), (keep, False),
                                     (0, True), (c - 1, True)):
            case = _Case(dtype, heads, kv_heads, dim, vdim, page, q_lens, [c], window, keep, seed=9)
            case.k[0] = torch.zeros_like(case.k[0])
            case.v[0] = torch.zeros_like(case.v[0])
            case.k[0][marked] = 4.0
            case.v[0][marked] = torch.arange(1, vdim + 1).to(dtype)
            case.q[0] = torch.ones_like(case.q[0])     # the marked key: 16 dims of 4 give 64, capped to 56, less 30: a weight of one
            out = case.run(ops, splits=1, **kw)
            torch.testing.assert_close(out, case.reference(**kw), **TOL[dtype])
            last = out[-1].view(heads, vdim)
            if seen_by_last:
                torch.testing.assert_close(last[0], torch.arange(1, vdim + 1, dtype=torch.float64), **TOL[dtype])
            else:
                assert float(last.abs().max()) < 1e-6


# ----------------------------------------------------------------------------- the linear memory

def _scan_inputs(mode, heads, dim, vdim, tokens, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    width = 2 * heads * dim + heads * vdim + 7              # columns the scan does not read lie behind
    x = (2.0 * torch.randn(tokens, width, generator=g)).to(dtype)
    g = torch.Generator().manual_seed(seed + 1000)          # gates that do not depend on the number of tokens
    extra = {}
    if mode == "gated_write":
        extra["lower"] = 1.0 - torch.logspace(-3, 0, heads * dim)[torch.randperm(heads * dim, generator=g)]
        extra["gate_bias"] = torch.randn(heads * dim, generator=g)
    else:
        extra["decay"] = torch.linspace(0.6, 1.0, heads)
    return x, extra


def _scan_reference(mode, x, extra, heads, dim, vdim):
    xd = x.double()
    T = xd.shape[0]
    q = plain.silu(xd[:, :heads * dim]).view(T, heads, dim)
    raw = xd[:, heads * dim:2 * heads * dim]
    v = xd[:, 2 * heads * dim:2 * heads * dim + heads * vdim].view(T, heads, vdim)
    if mode == "gated_write":
        low = extra["lower"].double()
        f = (low + (1.0 - low) * torch.sigmoid(raw + extra["gate_bias"].double())).view(T, heads, dim)
        return torch.cat([plain.decayed_memory(q[:, h], 1.0 - f[:, h], v[:, h], f[:, h]) for h in range(heads)], dim=-1)
    k = plain.silu(raw).view(T, heads, dim)
    v = plain.silu(v)
    return torch.cat([plain.decayed_memory(q[:, h], k[:, h], v[:, h], torch.full((T, dim), float(extra["decay"][h]),
                                                                                 dtype=torch.float64))
                      for h in range(heads)], dim=-1)


def _scan(ops, mode, x, extra, state, cu, slots, heads, dim, vdim):
    return ops.linear_scan(x.cuda(), state, _i32(cu), _i32(slots), num_heads=heads, head_dim=dim, v_dim=vdim, mode=mode,
                           q_off=0, k_off=heads * dim, v_off=2 * heads * dim,
                           **{k: v.float().cuda() for k, v in extra.items()}).double().cpu()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode", ["gated_write", "constant_decay"])
@pytest.mark.parametrize("heads,dim,vdim", [(3, 20, 12), (2, 8, 40), (1, 128, 128), (4, 64, 32), (2, 160, 48), (5, 1, 1)])
def test_linear_scan_whole_in_portions_and_token_by_token(dtype, mode, heads, dim, vdim):
    ops = _ops()
    lens = [45, 1, 23]
    floats = ops.linear_scan_state_floats(heads, dim, vdim)
    tol = dict(atol=3e-5, rtol=3e-5) if dtype == torch.float32 else dict(atol=2e-4, rtol=2e-4)   # inputs are exact in both
    xs, extras, wants = [], None, []
    for i, n in enumerate(lens):
        x, extras = _scan_inputs(mode, heads, dim, vdim, n, dtype, seed=7)       # the same gates for every sequence
        x = (x.float() * (0.5 + 0.5 * i)).to(dtype)
        xs.append(x)
        wants.append(_scan_reference(mode, x.float(), extras, heads, dim, vdim))
    # whole sequences in one step; the state lies in slots 4, 0, 2 of a wider state tensor (a share of a slot)
    state = torch.zeros((6, floats + 11), device="cuda")
    share = state[:, 3:3 + floats]
    slots = [4, 0, 2]
    cu = [0, 45, 46, 69]
    got = _scan(ops, mode, torch.cat(xs), extras, share, cu, slots, heads, dim, vdim)
    torch.testing.assert_close(got, torch.cat(wants), **tol)
    assert float(state[:, :3].abs().sum()) == 0.0 and float(state[:, 3 + floats:].abs().sum()) == 0.0
    assert float(state[[1, 3, 5]].abs().sum()) == 0.0
    whole = share.clone()
    # the same in portions of changing size (down to one token), sequences beside one another, a padded sequence
    # between them; then the memories are the same
    state2 = torch.zeros((6, floats + 11), device="cuda")
    share2 = state2[:, 3:3 + floats]
    done = [0, 0, 0]
    outs = [[], [], []]
    sizes = [(7, 1, 2), (1, 0, 1), (16, 0, 17), (2, 0, 1), (19, 0, 2)]
    for step in sizes:
        rows, cu2, sl = [], [0], []
        for s, n in enumerate(step):
            rows.append(xs[s][done[s]:done[s] + n])
            cu2.append(cu2[-1] + n)
            sl.append(slots[s] if n else -1)
        # a sequence without tokens in this step stands in as a padded one: a row of its own and slot -1
        rows = [r if r.shape[0] else xs[0][:1] for r in rows]
        cu2 = [0]
        for r in rows:
            cu2.append(cu2[-1] + r.shape[0])
        got = _scan(ops, mode, torch.cat(rows), extras, share2, cu2, sl, heads, dim, vdim)
        for s, n in enumerate(step):
            if n:
                outs[s].append(got[cu2[s]:cu2[s + 1]])
                done[s] += n
    assert done == lens
    for s in range(3):
        torch.testing.assert_close(torch.cat(outs[s]), wants[s], **tol)
    torch.testing.assert_close(share2, whole, atol=3e-5, rtol=3e-5)
    # the memory read back in plain order is the plain recurrence's
    if mode == "constant_decay":
        x = xs[1].double()
        k = plain.silu(x[0, heads * dim:2 * heads * dim]).view(heads, dim)
        v = plain.silu(x[0, 2 * heads * dim:2 * heads * dim + heads * vdim]).view(heads, vdim)
        want = k[:, :, None] * v[:, None, :]
        torch.testing.assert_close(ops.linear_scan_memory(share[0], heads, dim, vdim).double().cpu(), want, **tol)


def test_a_value_written_hundreds_of_tokens_back_is_still_read_and_a_reused_slot_starts_empty():
    ops = _ops()
    heads, dim, vdim, T = 1, 16, 32, 700
    floats = ops.linear_scan_state_floats(heads, dim, vdim)
    # gated write: row 0 never forgets (lower bound one), every other row forgets at once (gate zero)
    x = torch.zeros(T, 2 * dim + vdim)
    x[:, :dim] = 5.0                                           # q = silu(5) in every row
    x[:, dim:2 * dim] = -40.0                                  # sigmoid -> 0: f = lower
    x[3, 2 * dim:] = torch.arange(1, vdim + 1).float()         # written at token 3 only
    lower = torch.zeros(dim)
    lower[0] = 1.0 - 1e-3
    state = torch.zeros((2, floats), device="cuda")
    extra = {"lower": lower, "gate_bias": torch.zeros(dim)}
    outs = []
    for lo, hi in ((0, 2), (2, 300), (300, 301), (301, 699), (699, 700)):
        outs.append(_scan(ops, "gated_write", x[lo:hi], extra, state, [0, hi - lo], [1], heads, dim, vdim))
    out = torch.cat(outs)
    q = float(plain.silu(torch.tensor(5.0, dtype=torch.float64)))
    # row 0 took 1e-3 of the value at token 3 and keeps 0.999 of it per token; the other rows hold the newest value
    want_last = q * 1e-3 * (1.0 - 1e-3) ** (T - 1 - 3) * torch.arange(1, vdim + 1, dtype=torch.float64)
    torch.testing.assert_close(out[-1], want_last, atol=1e-7, rtol=2e-4)
    assert float(out[2].abs().max()) == 0.0
    # the slot is zeroed by whoever opens a request; a new sequence in it starts from nothing
    state[1].zero_()
    again = _scan(ops, "gated_write", x[:5], extra, state, [0, 5], [1], heads, dim, vdim)
    torch.testing.assert_close(again, out[:5], atol=1e-7, rtol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,group,full_weight,gated", [(36, 12, False, False), (60, 60, True, True), (512, 128, False, False),
                                                           (2048, 2048, True, True), (40, 40, False, True)])
def test_group_norm_gate(dtype, width, group, full_weight, gated):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(2)
    n, eps, factor = 19, 1e-5, 1.3
    o = 4.0 * torch.randn((n, width), generator=g, device="cuda")
    weight = 1.0 + 0.1 * torch.randn((width if full_weight else group,), generator=g, device="cuda")
    x = torch.randn((n, width + 9), generator=g, device="cuda").to(dtype) if gated else None
    got = ops.group_norm_gate(o, weight, group=group, eps=eps, out_dtype=dtype, factor=factor, x=x, gate_off=5)
    od = o.double().cpu().view(n, width // group, group)
    want = plain.rms_norm(od, None, eps).reshape(n, width) * weight.double().cpu().repeat(width // weight.numel()) * factor
    if gated:
        want = want * torch.sigmoid(x.double().cpu()[:, 5:5 + width])
    torch.testing.assert_close(got.double().cpu(), want, **TOL[dtype])


# ----------------------------------------------------------------------------- the pair table and the stream

@pytest.mark.parametrize("dtype", DTYPES)
def test_pair_rows_across_steps_with_the_previous_token_in_the_state(dtype):
    ops = _ops()
    vocab, hidden, buckets, mp, mc = 50, 24, 13, 7, 3
    g = torch.Generator().manual_seed(1)
    table = torch.randn(buckets + 1, hidden, generator=g).to(dtype)
    embed = torch.randn(vocab, hidden, generator=g).to(dtype)
    seqs = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (9, 1, 14)]
    raw = {"embedding": {"scale": 2.0, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    w = {"embed": embed.double(), "bigram": table.double()}
    wants = [plain.embed(s, w, raw) for s in seqs]
    last = torch.zeros((5, 3), dtype=torch.int32, device="cuda")         # a wider state: the token is its first entry
    slots = [3, 0, 4]
    done, outs = [0, 0, 0], [[], [], []]
    sampled = torch.zeros(4, dtype=torch.int32, device="cuda")
    for step in ((4, 1, 1), (1, 0, 1), (2, 0, 10), (2, 0, 2)):
        ids, pos, cu, sl = [], [], [0], []
        for s, n in enumerate(step):
            if not n:
                continue
            ids += seqs[s][done[s]:done[s] + n]
            pos += list(range(done[s], done[s] + n))
            cu.append(cu[-1] + n)
            sl.append(slots[s])
        # one token of the step is named by the row of the choices it was made in, not by its id
        sampled[2] = ids[-1]
        ids_dev = _i32(ids[:-1] + [-3])
        hidden_rows = ops.embedding(ids_dev, embed.cuda(), sampled=sampled, scale=2.0)
        ops.pair_rows_add(hidden_rows, ids_dev, _i32(pos), _i32(cu), _i32(sl), last, table.cuda(), vocab=vocab,
                          buckets=buckets, mul_prev=mp, mul_cur=mc, sampled=sampled)
        at = 0
        for s, n in enumerate(step):
            if n:
                outs[s].append(hidden_rows[at:at + n].double().cpu())
                at += n
                done[s] += n
    for s in range(3):
        torch.testing.assert_close(torch.cat(outs[s]), wants[s], atol=1e-6, rtol=1e-6)
    assert [int(last[slot, 0]) for slot in slots] == [seq[-1] for seq in seqs]
    assert int(last[:, 1:].abs().sum()) == 0 and int(last[[1, 2]].abs().sum()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_add_and_scaled_sum(dtype):
    ops = _ops()
    g = torch.Generator(device="cuda").manual_seed(3)
    for shape in ((5, 72), (3, 7), (33, 256)):
        hidden = torch.randn(shape, generator=g, device="cuda")
        other = torch.randn(shape, generator=g, device="cuda")
        want = hidden + other
        pending = torch.ones(shape, device="cuda", dtype=dtype)
        assert ops.stream_add(hidden, other, pending) is pending
        torch.testing.assert_close(hidden, want, atol=0, rtol=0)
        a, b = torch.randn(shape, generator=g, device="cuda").to(dtype), torch.randn(shape, generator=g, device="cuda").to(dtype)
        torch.testing.assert_close(ops.scaled_sum(a, b, 0.8, 1.1).double(), (a.double() * 0.8 + b.double() * 1.1),
                                   **TOL[dtype])
    assert ops.stream_add(hidden, other, ops.Summed(hidden, other)) is None
