"""The kernels that came with the Zavizen design, each alone, against plain formulas (float64), in float32 and bfloat16
storage: the stream in several copies (write, read and norm in one pass, the collapse, gathered rows); two branch
outputs normed and summed; the rotation with norms over the whole q and k rows and the cache write; float32 rows for a
scan; the linear-memory scan on prepared rows with a constant decay and with a decay per token and shared q/k heads
(whole, in portions down to one token, through state slots that are used again, a value written hundreds of tokens
back); the state-space preparation with its convolution across step borders; the norm with a skip term and a gate
before it; routing with softmax scores and groups scored by their best expert; the experts' plain SiLU."""

import pytest
import torch

from plain import zavizen_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: dict(atol=2e-5, rtol=2e-5), torch.bfloat16: dict(atol=2e-2, rtol=2e-2)}


def _ops():
    from ampere_kv_engine_b200.kernels import ops
    return ops


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return scale * torch.randn(shape, generator=g, device="cuda")


# ----------------------------------------------------------------------------- the stream in several copies

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("streams,width,y_float", [(1, 40, True), (3, 72, False), (4, 256, True), (8, 1031, False),
                                                   (2, 2048, False), (5, 4100, True)])
def test_hyper_step_collapse_and_expand(dtype, streams, width, y_float):
    ops = _ops()
    n, eps = 13, 1e-5
    row = _rand((n, width), 1, 3.0)
    x = ops.hyper_expand(row, streams)
    assert x.shape == (n, streams, width) and all(torch.equal(x[:, s], row) for s in range(streams))
    x = x + _rand(x.shape, 2)
    mix, write, read = _rand((streams, streams), 3), _rand((streams,), 4), _rand((streams,), 5)
    scale, weight = 1.0 + _rand((width,), 6, 0.1), 1.0 + _rand((width,), 7, 0.1)
    y = _rand((n, width), 8).to(torch.float32 if y_float or dtype == torch.float32 else dtype)
    new = torch.einsum("st,nsw->ntw", mix.double(), x.double()) + write.double()[None, :, None] * \
        (y.double() * scale.double())[:, None, :]
    u = torch.einsum("s,nsw->nw", read.double(), new)
    want = plain.rms_norm(u, weight.double(), eps)
    pending = ops.HyperPending(y, mix, write, scale)
    torch.testing.assert_close(ops.hyper_collapse(x.clone(), pending).double(), new.sum(1), atol=1e-4, rtol=1e-5)
    torch.testing.assert_close(ops.hyper_collapse(x.clone(), None).double(), x.double().sum(1), atol=1e-4, rtol=1e-5)
    work = x.clone()
    got = ops.hyper_step(work, pending, read, weight, eps, dtype)
    torch.testing.assert_close(work.double(), new, atol=1e-4, rtol=1e-5)
    torch.testing.assert_close(got.double(), want, **TOL[dtype])
    # a read alone leaves the copies as they are; gathered rows
    again = ops.hyper_step(work, None, read, weight, eps, dtype)
    torch.testing.assert_close(again, got)
    rows = _i32([n - 1, 0, 5])
    torch.testing.assert_close(ops.hyper_step(work, None, read, weight, eps, dtype, rows=rows), got[rows.long()])
    # a write alone
    work2 = x.clone()
    assert ops.hyper_step(work2, ops.HyperPending(y, mix, write, None), None, None, eps, dtype) is None
    plain_new = torch.einsum("st,nsw->ntw", mix.double(), x.double()) + write.double()[None, :, None] * y.double()[:, None, :]
    torch.testing.assert_close(work2.double(), plain_new, atol=1e-4, rtol=1e-5)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.hyper_step(work, None, read, weight, eps, dtype, rows=_i32([n]), status=status)
    assert int(status) != 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_normed_pair_sum(dtype):
    ops = _ops()
    a, b = _rand((9, 200), 1, 5.0), _rand((9, 200), 2, 0.01)
    wa, wb = _rand((200,), 3), _rand((200,), 4)
    want = 0.5 * plain.rms_norm(a.double(), wa.double(), 1e-6) + 0.25 * plain.rms_norm(b.double(), wb.double(), 1e-6)
    got = ops.normed_pair_sum(a, b, wa, wb, eps=1e-6, sa=0.5, sb=0.25, out_dtype=dtype)
    torch.testing.assert_close(got.double(), want, **TOL[dtype])


# ----------------------------------------------------------------------------- rotation with norms over whole rows

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rot_dims,factor", [
    (4, 2, 24, 16, 16, 2.0), (6, 1, 128, 64, 48, 8.0), (3, 3, 20, 12, 4, None), (1, 1, 32, 40, 32, None)])
def test_rotary_prep_with_norms_over_the_whole_projections(dtype, heads, kv_heads, dim, vdim, rot_dims, factor):
    ops = _ops()
    from ampere_kv_engine_b200.config.spec import PartSpec
    from ampere_kv_engine_b200.parts.base import POSITION_ENCODINGS, build_part
    n, page_size, pages, eps = 41, 8, 9, 1e-5
    rot = {"dims": rot_dims, "base": 500.0}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    rope = build_part(POSITION_ENCODINGS, PartSpec("rope", {"theta": 500.0, "rotary_dim": rot_dims, "layout": "half",
                                                           "scaling": rot.get("scaling") or {"factor": 1.0}}),
                      hidden_size=8, dtype=dtype, device=torch.device("cuda"))
    freq, dims, layout, cs = rope.rotary_table()
    assert torch.equal(freq.cpu(), plain.rotary_frequencies(rot).float())
    assert cs == 1.0 and layout == "half"
    g = torch.Generator(device="cuda").manual_seed(5)
    x = (3.0 * torch.randn((n, (heads + kv_heads) * dim + kv_heads * vdim), generator=g, device="cuda")).to(dtype)
    positions = torch.randint(0, 3000, (n,), generator=g, device="cuda").to(torch.int32)
    slots = torch.randperm(pages * page_size, generator=g, device="cuda")[:n].to(torch.int32)
    qw, kw = 1.0 + _rand((heads * dim,), 6, 0.3), 1.0 + _rand((kv_heads * dim,), 7, 0.3)
    k_cache = torch.zeros((pages, kv_heads, page_size, dim), dtype=dtype, device="cuda")
    v_cache = torch.zeros((pages, kv_heads, page_size, vdim), dtype=dtype, device="cuda")
    q = ops.rotary_prep(x, positions, slots, freq, k_cache, v_cache, num_heads=heads, num_kv_heads=kv_heads,
                        head_dim=dim, v_dim=vdim, rotary_dims=rot_dims, layout="half", q_norm=qw, k_norm=kw,
                        row_norm_eps=eps)
    xd = x.double().cpu()
    a, b = heads * dim, kv_heads * dim

    def turned(rows, weight, count):
        rows = plain.rms_norm(rows, weight.double().cpu(), eps).view(n, count, dim)
        out = torch.empty_like(rows)
        for t in range(n):
            out[t] = plain.rotate_half(rows[t:t + 1], rot, first=int(positions[t]))[0]
        return out

    torch.testing.assert_close(q.double().cpu(), turned(xd[:, :a], qw, heads).reshape(n, -1), **TOL[dtype])
    s = slots.long().cpu()
    torch.testing.assert_close(k_cache.double().cpu()[s // page_size, :, s % page_size], turned(xd[:, a:a + b], kw, kv_heads),
                               **TOL[dtype])
    torch.testing.assert_close(v_cache.double().cpu()[s // page_size, :, s % page_size],
                               xd[:, a + b:].view(n, kv_heads, vdim), **TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim,rot_dims", [(3, 12, 20, 12), (2, 64, 32, 32), (1, 24, 9, 8)])
def test_rotary_rows(dtype, heads, dim, vdim, rot_dims):
    ops = _ops()
    n = 17
    rot = {"dims": rot_dims, "base": 100.0}
    freq = plain.rotary_frequencies(rot).float().cuda()
    qk, vw = heads * dim, heads * vdim
    x = _rand((n, 2 * qk + 2 * vw), 3, 2.0).to(dtype)
    positions = _i32(list(range(100, 100 + n)))
    rows = ops.rotary_rows(x, positions, freq, num_heads=heads, head_dim=dim, v_dim=vdim, rotary_dims=rot_dims, q_off=0,
                           k_off=qk, v_off=2 * qk, k_scale=dim ** -0.5)
    assert rows.dtype == torch.float32 and rows.shape[1] % 4 == 0 and rows.shape[1] >= 2 * qk + vw
    xd = x.double().cpu()
    want_q = plain.rotate_half(xd[:, :qk].view(n, heads, dim), rot, first=100).reshape(n, -1)
    want_k = plain.rotate_half(xd[:, qk:2 * qk].view(n, heads, dim), rot, first=100).reshape(n, -1) * dim ** -0.5
    torch.testing.assert_close(rows[:, :qk].double().cpu(), want_q, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(rows[:, qk:2 * qk].double().cpu(), want_k, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(rows[:, 2 * qk:2 * qk + vw].double().cpu(), xd[:, 2 * qk:2 * qk + vw], atol=0, rtol=0)


# ----------------------------------------------------------------------------- the scan on prepared rows

def _scan_reference(q, k, v, decay):
    """q, k [T, H, D], v [T, H, V], decay [T, H] float64 -> o [T, H, V] and the last memory [H, D, V]."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2], dtype=torch.float64)
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for t in range(T):
        S = decay[t][:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out, S


@pytest.mark.parametrize("mode", ["plain_decay", "token_decay"])
@pytest.mark.parametrize("heads,group,dim,vdim", [(3, 1, 12, 20), (4, 2, 20, 12), (2, 1, 64, 32), (6, 3, 40, 56),
                                                  (2, 2, 130, 40), (1, 1, 7, 5), (4, 4, 128, 64)])
def test_scan_whole_in_portions_and_token_by_token(mode, heads, group, dim, vdim):
    ops = _ops()
    if mode == "plain_decay":
        group = 1
    T = 77
    qh = heads // group
    qk, vw = qh * dim, heads * vdim
    width = (2 * qk + vw + heads + 3) // 4 * 4
    rows = _rand((T, width), 11, 0.5)
    per_token = torch.rand((T, heads), generator=torch.Generator(device="cuda").manual_seed(12), device="cuda") * 0.5 + 0.5
    rows[:, 2 * qk + vw:2 * qk + vw + heads] = per_token
    fixed = torch.tensor([1.0 - 0.5 ** (i + 1) for i in range(heads)], device="cuda")
    rd = rows.double().cpu()
    q = rd[:, :qk].view(T, qh, dim).repeat_interleave(group, 1)
    k = rd[:, qk:2 * qk].view(T, qh, dim).repeat_interleave(group, 1)
    v = rd[:, 2 * qk:2 * qk + vw].view(T, heads, vdim)
    decay = per_token.double().cpu() if mode == "token_decay" else fixed.double().cpu()[None, :].expand(T, heads)
    want, last = _scan_reference(q, k, v, decay)
    floats = ops.linear_scan_state_floats(heads, dim, vdim)
    kw = dict(num_heads=heads, head_dim=dim, v_dim=vdim, mode=mode, q_off=0, k_off=qk, v_off=2 * qk,
              decay=fixed if mode == "plain_decay" else None, qk_group=group, decay_off=2 * qk + vw)
    for cuts in ([T], [1] * T, [30, 2, 1, 7, 2, 35], [2] * 38 + [1]):
        # a state wider than the memory (another mixer's share behind it), slot 2 of 4, NaN elsewhere
        state = torch.full((4, floats + 8), float("nan"), device="cuda")
        state[2] = 0.0
        outs, at = [], 0
        for n in cuts:
            outs.append(ops.linear_scan(rows[at:at + n].contiguous(), state, _i32([0, n]), _i32([2]), **kw))
            at += n
        got = torch.cat(outs).double().cpu().view(T, heads, vdim)
        torch.testing.assert_close(got, want, atol=2e-5, rtol=2e-5)
        torch.testing.assert_close(ops.linear_scan_memory(state[2], heads, dim, vdim).double().cpu(), last, atol=2e-5, rtol=2e-5)
        assert torch.isnan(state[[0, 1, 3]]).all() and not torch.isnan(state[2, floats:]).any()
    # three sequences of unequal length in one step, one of them padding (slot -1), against each alone
    state = torch.zeros((4, floats), device="cuda")
    both = ops.linear_scan(rows[:60].contiguous(), state, _i32([0, 40, 41, 60]), _i32([3, -1, 0]), **kw)
    for lo, hi, slot in ((0, 40, 3), (41, 60, 0)):
        alone = torch.zeros((1, floats), device="cuda")
        one = ops.linear_scan(rows[lo:hi].contiguous(), alone, _i32([0, hi - lo]), _i32([0]), **kw)
        torch.testing.assert_close(both[lo:hi], one, atol=1e-6, rtol=1e-6)
        torch.testing.assert_close(state[slot], alone[0], atol=1e-6, rtol=1e-6)


def test_a_value_written_hundreds_of_tokens_back_is_still_read():
    ops = _ops()
    heads, dim, vdim, T = 2, 16, 8, 640
    qk, vw = heads * dim, heads * vdim
    width = 2 * qk + vw + 4
    rows = torch.zeros((T, width), device="cuda")
    rows[:, 2 * qk + vw] = 1.0                    # head 0 never forgets
    rows[:, 2 * qk + vw + 1] = 0.995              # head 1 fades
    rows[3, qk + 5] = rows[3, qk + dim + 5] = 2.0                 # token 3 writes row 5 of both heads
    rows[3, 2 * qk:2 * qk + vw] = torch.arange(1, vw + 1, device="cuda").float()
    rows[T - 1, 5] = rows[T - 1, dim + 5] = 1.0                   # the last token reads row 5
    state = torch.zeros((1, ops.linear_scan_state_floats(heads, dim, vdim)), device="cuda")
    kw = dict(num_heads=heads, head_dim=dim, v_dim=vdim, mode="token_decay", q_off=0, k_off=qk, v_off=2 * qk,
              decay_off=2 * qk + vw)
    out = ops.linear_scan(rows[:600].contiguous(), state, _i32([0, 600]), _i32([0]), **kw)
    assert float(out[4:].abs().max()) == 0.0
    for t in range(600, T):
        out = ops.linear_scan(rows[t:t + 1].contiguous(), state, _i32([0, 1]), _i32([0]), **kw)
    want = 2.0 * torch.arange(1, vw + 1).float().view(heads, vdim)
    want[1] *= 0.995 ** (T - 1 - 3)
    torch.testing.assert_close(out.view(heads, vdim).cpu(), want, atol=1e-4, rtol=1e-4)


# ----------------------------------------------------------------------------- the state-space preparation

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,vdim,state_dim,groups,taps", [(4, 12, 20, 2, 3), (2, 40, 8, 1, 2), (3, 16, 12, 3, 1),
                                                            (6, 8, 36, 2, 5)])
def test_ssm_prep_and_the_convolution_across_step_borders(dtype, heads, vdim, state_dim, groups, taps):
    ops = _ops()
    T = 23
    inner, gn = heads * vdim, groups * state_dim
    channels = inner + 2 * gn
    in_width = 2 * inner + 2 * gn + heads
    x = _rand((T, in_width), 21, 1.5).to(dtype)
    conv, bias = _rand((channels, taps), 22, 0.5), _rand((channels,), 23, 0.3)
    step_bias, rate_log = _rand((heads,), 24), _rand((heads,), 25, 0.5)
    xd = x.double().cpu()
    y = plain.silu(plain.short_convolution(xd[:, inner:inner + channels], conv.double().cpu(), bias.double().cpu()))
    dt = plain.softplus(xd[:, inner + channels:] + step_bias.double().cpu())
    decay = torch.exp(-torch.exp(rate_log.double().cpu()) * dt)
    want = torch.cat((y[:, inner + gn:], y[:, inner:inner + gn], y[:, :inner] * dt.repeat_interleave(vdim, 1), decay,
                      y[:, :inner]), dim=1)
    memory = 40                                           # the tail lives behind another 40 floats of the slot
    floats = memory + (taps - 1) * channels
    kw = dict(tail_off=memory, num_heads=heads, v_dim=vdim, state_dim=state_dim, groups=groups, taps=taps,
              conv_off=inner, step_off=inner + channels)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=1e-4, rtol=1e-4)   # x itself is exact
    for cuts in ([T], [1] * T, [5, 2, 1, 1, 3, 2, 9], [2] * 11 + [1]):
        state = torch.full((3, floats + 4), float("nan"), device="cuda")
        state[1] = 0.0
        outs, at = [], 0
        for n in cuts:
            part = x[at:at + n].contiguous()
            outs.append(ops.ssm_prep(part, conv, bias, step_bias, rate_log, state, _i32([0, n]), _i32([1]), **kw))
            ops.conv_tail(part, state, _i32([0, n]), _i32([1]), tail_off=memory, conv_off=inner, channels=channels, taps=taps)
            at += n
        got = torch.cat(outs)[:, :want.shape[1]].double().cpu()
        torch.testing.assert_close(got, want, **tol)
        assert float(state[1, :memory].abs().max()) == 0.0 and torch.isnan(state[[0, 2]]).all()
        if taps > 1:
            kept = state[1, memory:memory + (taps - 1) * channels].view(taps - 1, channels).double().cpu()
            torch.testing.assert_close(kept, xd[T - (taps - 1):, inner:inner + channels], atol=0, rtol=0)
    # a padded sequence's rows are zero and its (absent) slot is left alone
    state = torch.zeros((2, floats + 4), device="cuda")
    out = ops.ssm_prep(x[:6].contiguous(), conv, bias, step_bias, rate_log, state, _i32([0, 4, 6]), _i32([0, -1]), **kw)
    assert float(out[4:6, :want.shape[1]].abs().max()) == 0.0 and float(out[:4, :want.shape[1]].abs().max()) > 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,group,head,weighted,gate,first,skip", [
    (48, 24, 12, True, "silu", True, True), (80, 80, 40, True, "silu", True, True),
    (60, 20, 20, False, "silu", False, False), (64, 64, 16, True, "sigmoid", False, False),
    (36, 12, 12, False, None, False, True)])
def test_group_norm_gate_with_a_skip_term_and_either_gate(dtype, width, group, head, weighted, gate, first, skip):
    ops = _ops()
    n, eps = 11, 1e-5
    o = _rand((n, width), 31, 2.0)
    weight = (1.0 + _rand((width,), 32, 0.2)) if weighted else None
    x = _rand((n, width + 9), 33).to(dtype)
    extra = _rand((n, width + 5), 34)
    coef = _rand((width // head,), 35)
    v = o.double().cpu()
    if skip:
        v = v + extra[:, 5:].double().cpu() * coef.double().cpu().repeat_interleave(head)
    z = x[:, 9:].double().cpu()
    gv = None if gate is None else (plain.silu(z) if gate == "silu" else torch.sigmoid(z))
    if gv is not None and first:
        v = v * gv
    want = plain.rms_norm(v.view(n, width // group, group), None, eps).reshape(n, width)
    if weighted:
        want = want * weight.double().cpu()
    if gv is not None and not first:
        want = want * gv
    got = ops.group_norm_gate(o, weight, group=group, eps=eps, out_dtype=dtype, x=x if gate else None, gate_off=9,
                              gate=gate or "sigmoid", gate_first=first, skip=extra if skip else None, skip_off=5,
                              skip_coef=coef if skip else None, skip_head=head)
    torch.testing.assert_close(got.double().cpu(), want, **TOL[dtype])


# ----------------------------------------------------------------------------- routing and the experts' activation

@pytest.mark.parametrize("experts,top,groups,keep", [(10, 4, 2, 1), (6, 2, 3, 2), (4, 1, 1, 1), (3, 3, 1, 1), (64, 6, 8, 3)])
def test_softmax_routing_with_groups_scored_by_their_best_expert(experts, top, groups, keep):
    ops = _ops()
    logits = _rand((50, experts), 41, 3.0)
    router = {"experts": experts, "top": top, "scale": 1.75, "groups": {"count": groups, "keep": keep}}
    want_ids, want_w = plain.route(logits.double().cpu(), router)
    chosen, weights = ops.moe_route(logits, None, top=top, groups=groups, keep_groups=keep, group_top=1, scale=1.75,
                                    weight_eps=1e-20, score="softmax")
    order = want_ids.sort(dim=1)
    got = chosen.long().cpu().sort(dim=1)
    assert torch.equal(got.values, order.values)
    torch.testing.assert_close(weights.double().cpu().gather(1, got.indices), want_w.gather(1, order.indices),
                               atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(weights.sum(1).cpu(), torch.full((50,), 1.75), atol=1e-5, rtol=1e-5)


def test_a_group_of_one_very_good_expert_beats_a_group_of_two_good_ones():
    ops = _ops()
    # groups {0, 1}, {2, 3}: the sum of the first group's scores is larger, the best expert sits in the second
    logits = torch.tensor([[2.0, 2.0, 2.5, -3.0]], device="cuda")
    chosen, weights = ops.moe_route(logits, None, top=2, groups=2, keep_groups=1, group_top=1, scale=1.0,
                                    weight_eps=1e-20, score="softmax")
    assert sorted(chosen[0].tolist()) == [2, 3]
    s = torch.softmax(logits[0].double().cpu(), -1)
    torch.testing.assert_close(weights[0].double().cpu().sort().values, (s[[3, 2]] / (s[2] + s[3])), atol=1e-6, rtol=1e-5)
    # very negative logits everywhere: the scores underflow towards zero in all but the best, the choice still stands
    logits = torch.tensor([[-80.0, -200.0, -90.0, -300.0]], device="cuda")
    chosen, weights = ops.moe_route(logits, None, top=2, groups=1, keep_groups=1, group_top=1, scale=2.0,
                                    weight_eps=1e-20, score="softmax")
    assert chosen[0].tolist() == [0, 2] and float(weights.sum()) == pytest.approx(2.0, rel=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kernel", ["auto", "plain", "mma", "few"])
def test_experts_with_plain_silu(dtype, kernel):
    ops = _ops()
    if dtype == torch.float32 and kernel in ("mma", "few"):
        pytest.skip("the tensor-core and few-rows forms are bfloat16")
    experts, top, hidden, inter, n = 5, 2, 64, 24, 19
    x = _rand((n, hidden), 51).to(dtype)
    w_gu = _rand((experts, 2 * inter, hidden), 52, 0.2).to(dtype)
    w_d = _rand((experts, hidden, inter), 53, 0.2).to(dtype)
    chosen = torch.stack([torch.randperm(experts, generator=torch.Generator().manual_seed(i))[:top] for i in range(n)])
    chosen = chosen.to(torch.int32).cuda()
    weights = torch.rand((n, top), generator=torch.Generator().manual_seed(9)).cuda()
    order, offsets = ops.moe_sort(chosen, experts)
    act = ops.moe_gate_up(x, w_gu, order, offsets, top=top, limit=float("inf"), slope=1.0, up_offset=0.0, kernel=kernel)
    parts = ops.moe_down(act, w_d, order, offsets, weights, kernel=kernel if kernel != "few" else "auto")
    got = ops.moe_combine(parts, None, top=top)
    want = torch.zeros(n, hidden, dtype=torch.float64)
    xd, gu, dn = x.double().cpu(), w_gu.double().cpu(), w_d.double().cpu()
    for t in range(n):
        for c in range(top):
            e = int(chosen[t, c])
            h = plain.silu(xd[t] @ gu[e, :inter].T) * (xd[t] @ gu[e, inter:].T)
            if dtype == torch.bfloat16:
                h = h.to(torch.bfloat16).double()
            want[t] += float(weights[t, c]) * (h @ dn[e].T)
    torch.testing.assert_close(got.double().cpu(), want, **(dict(atol=2e-4, rtol=2e-4) if dtype == torch.float32 else
                                                          dict(atol=3e-2, rtol=3e-2)))
