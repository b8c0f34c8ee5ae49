"""The kernels and part options that Bogetar added, each against the plain function of the same mechanism
(float64 on the CPU), on sizes the tiny models do not reach, cut into portions and decoded, over hand-made paged
caches and state slots, with inputs made so that a fault shows: a key that stands out just inside and just
outside a window (every other key's weight pushed to nothing by the head's bias), a far write of a recurrence
read back after hundreds of tokens, slots that are used again."""

import math

import pytest
import torch

import plain_bogetar as pb

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def F():
    from mini_infer_b200.ops import functional
    return functional


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def close(got, want, tol):
    return float((got.double().cpu() - want).abs().max()) <= tol * max(float(want.abs().max()), 1e-30)


# --------------------------------------------------------------------------- #
# norms in groups
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("T,W,groups", [(1, 40, 1), (7, 192, 2), (5, 48, 3), (3, 1026, 2), (2, 4100, 5), (4, 8192, 1),
                                        (3, 33, 11), (2, 3072, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_in_groups(T, W, groups, dtype):
    g = torch.Generator().manual_seed(T + W)
    x, w = torch.randn(T, W, generator=g) * 3, 1 + 0.3 * torch.randn(W, generator=g)
    want = pb.group_rms_norm(x.double(), w.double(), groups, 1e-5)
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    assert close(F().group_rmsnorm(x.to(DEV), w.to(DEV), groups, 1e-5, dtype), want, tol)
    rows = [T - 1, 0]
    assert close(F().group_rmsnorm(x.to(DEV), w.to(DEV), groups, 1e-5, dtype, i32(rows)), want[rows], tol)


@pytest.mark.parametrize("T,W,groups", [(1, 40, 1), (7, 192, 2), (5, 48, 3), (3, 1026, 2), (2, 4100, 5), (3, 33, 11),
                                        (2, 3072, 2), (2, 6000, 3)])
def test_output_norm_in_groups_added_to_the_residual(T, W, groups):
    g = torch.Generator().manual_seed(3 * T + W)
    hidden, y = torch.randn(T, W, generator=g), torch.randn(T, W, generator=g) * 2
    w = 1 + 0.3 * torch.randn(W, generator=g)
    want = hidden.double() + pb.group_rms_norm(y.double(), w.double(), groups, 1e-6)
    h = hidden.to(DEV)
    F().out_norm_add(h, y.to(DEV), w.to(DEV), 1e-6, 1.0, None, groups=groups)
    assert close(h, want, 3e-6)
    # the same row as a sum of rows formed inside the kernel: a * rows[t] + b * extra[t], and experts' rows by index
    a, b = 0.6, 0.9
    y2 = torch.randn(T, W, generator=g)
    h = hidden.to(DEV)
    F().out_norm_add(h, (y.to(DEV), None, torch.full((T, 1), a, device=DEV), y2.to(DEV), torch.full((T,), b, device=DEV)),
                     w.to(DEV), 1e-6, 1.0, None, groups=groups)
    want = hidden.double() + pb.group_rms_norm(a * y.double() + b * y2.double(), w.double(), groups, 1e-6)
    assert close(h, want, 3e-6)
    K = 3
    rows = torch.randn(T * K, W, generator=g)
    index = torch.randperm(T * K, generator=g).to(torch.int32).view(T, K)
    wk = torch.rand(T, K, generator=g)
    h = hidden.to(DEV)
    F().out_norm_add(h, (rows.to(DEV), index.to(DEV), wk.to(DEV), None, None), w.to(DEV), 1e-6, 1.0, None, groups=groups)
    summed = (rows.double()[index.long()] * wk.double()[:, :, None]).sum(dim=1)
    assert close(h, hidden.double() + pb.group_rms_norm(summed, w.double(), groups, 1e-6), 3e-6)


# --------------------------------------------------------------------------- #
# x + conv(x) with the last rows kept per request
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("C,taps", [(48, 3), (192, 4), (40, 1), (33, 2), (1024, 4), (70, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_input_convolution_in_portions_and_batches(C, taps, dtype):
    """Three requests of unequal length, fed in portions of changing size side by side, in slots that a request
    before them has used; every portion's first rows read the state that the portion before left."""
    g = torch.Generator().manual_seed(C + taps)
    w = torch.randn(C, taps, generator=g) * 0.5
    lens = [37, 5, 18]
    xs = [torch.randn(n, C, generator=g) for n in lens]
    want = [x.double() + pb.causal_conv(x.double(), w.double()) for x in xs]
    floats = max((taps - 1) * C, 1)
    state = torch.randn(5, floats + 3, generator=g).to(DEV)          # rows wider than the section, and dirty
    slots = [3, 0, 4]
    state[slots, 3:] = 0.0                                            # a new request's slot is zeroed
    cuts = [[1, 2, 7, 1, 1, 20, 5], [2, 1, 1, 1], [9, 2, 2, 5]]
    fed = [0, 0, 0]
    got = [[] for _ in lens]
    for step in range(7):
        live = [r for r in range(3) if step < len(cuts[r])]
        rows = [xs[r][fed[r]:fed[r] + cuts[r][step]] for r in live]
        x = torch.cat(rows).to(DEV)
        starts = [0]
        for r in rows:
            starts.append(starts[-1] + r.shape[0])
        req = [i for i, r in enumerate(rows) for _ in range(r.shape[0])]
        out = F().causal_conv_residual(x, w.to(DEV), state, 3, i32(starts), i32(req), i32([slots[r] for r in live]), dtype)
        for i, r in enumerate(live):
            got[r].append(out[starts[i]:starts[i + 1]].cpu())
            fed[r] += cuts[r][step]
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    for r in range(3):
        assert fed[r] == lens[r] and close(torch.cat(got[r]), want[r], tol), r
    assert bool((state[:, :3].cpu() != 0).all())                      # what lies before the section is left alone


@pytest.mark.parametrize("C,taps,groups", [(48, 3, 3), (192, 4, 2), (40, 1, 1), (33, 2, 11), (1024, 4, 2), (70, 8, 5)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_convolution_and_state_of_a_decode_step_in_one_launch(C, taps, groups, dtype):
    """Four requests decode twelve tokens each, one token per request and step, after a prompt portion that went
    through the kernels of any step; slots in another order than the requests."""
    g = torch.Generator().manual_seed(C + taps)
    w, nw = torch.randn(C, taps, generator=g) * 0.5, 1 + 0.3 * torch.randn(C, generator=g)
    B, first, more = 4, [5, 1, 9, 2], 12
    xs = [torch.randn(n + more, C, generator=g) * 2 for n in first]
    normed = [pb.group_rms_norm(x.double(), nw.double(), groups, 1e-5) for x in xs]
    want = [n + pb.causal_conv(n, w.double()) for n in normed]
    state = torch.zeros(6, max((taps - 1) * C, 1), device=DEV)
    slots = [4, 1, 0, 3]
    got = [[] for _ in range(B)]
    rows = torch.cat([x[:n] for x, n in zip(xs, first)]).to(DEV)
    starts = [0]
    for n in first:
        starts.append(starts[-1] + n)
    req = [i for i, n in enumerate(first) for _ in range(n)]
    n32 = F().group_rmsnorm(rows, nw.to(DEV), groups, 1e-5, torch.float32)
    out = F().causal_conv_residual(n32, w.to(DEV), state, 0, i32(starts), i32(req), i32(slots), dtype)
    for i in range(B):
        got[i].append(out[starts[i]:starts[i + 1]].cpu())
    for step in range(more):
        rows = torch.stack([xs[i][first[i] + step] for i in range(B)]).to(DEV)
        out = F().norm_conv_decode(rows, nw.to(DEV), groups, 1e-5, w.to(DEV), state, 0, i32(list(range(B + 1))),
                                   i32(slots), dtype)
        for i in range(B):
            got[i].append(out[i:i + 1].cpu())
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    for i in range(B):
        assert close(torch.cat(got[i]), want[i], tol), i
    assert float(state[[2, 5]].abs().sum()) == 0.0 or taps == 1          # slots of no request are left alone


# --------------------------------------------------------------------------- #
# the two recurrences on the walk of the delta rule
# --------------------------------------------------------------------------- #

def plain_delta(q, k, v, beta, decay):
    """q, k [T, H, d] as the walk reads them, v [T, H, dv], beta [T, H] or None (no correction), decay [T, H, d]."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=torch.float64)
    out = []
    for t in range(T):
        S = decay[t][:, :, None] * S
        u = v[t] if beta is None else beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out), S


def walk(form, qkv, beta, a, a_log, bias, H, G, d, dv, scale, cuts, tau=1.0, slot=1, segment_tokens=0):
    """``segment_tokens``: portions longer than that are walked in segments of so many tokens side by side."""
    T = qkv.shape[0]
    state = torch.randn(3, H * d * dv + 5, generator=torch.Generator().manual_seed(1)).to(DEV)
    state[slot, :H * d * dv] = 0.0
    outs, lo = [], 0
    for n in cuts:
        segs = -(-n // segment_tokens) if segment_tokens and n > segment_tokens else 1
        outs.append(F().delta_scan(qkv[lo:lo + n].to(DEV).contiguous(), None if beta is None else beta[lo:lo + n].to(DEV).contiguous(),
                                   0, a[lo:lo + n].to(DEV).contiguous(), 0, None if a_log is None else a_log.to(DEV),
                                   bias.to(DEV), state, 0, i32([0, n]), i32([slot]), H, G, d, dv, scale, form=form, tau=tau,
                                   segments=segs, segment_tokens=segment_tokens if segs > 1 else 0))
        lo += n
    assert lo == T
    return torch.cat(outs).cpu(), state[slot, :H * d * dv].cpu().view(H, d, dv)


@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 12, 10), (2, 2, 64, 64), (6, 1, 100, 24), (1, 1, 8, 8), (3, 3, 200, 17)])
def test_delta_rule_with_one_decay_per_head(H, G, d, dv):
    g = torch.Generator().manual_seed(H * d)
    T = 45
    qkv = torch.randn(T, 2 * G * d + H * dv + 7, generator=g)          # rows that go on with columns nobody reads
    beta, a = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g)
    a_log, bias = torch.randn(H, generator=g) * 0.5 - 1, torch.randn(H, generator=g)
    x = qkv.double()
    q, k = x[:, :G * d].view(T, G, d), x[:, G * d:2 * G * d].view(T, G, d)
    q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5).repeat_interleave(H // G, dim=1)
    k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(H // G, dim=1)
    v = x[:, 2 * G * d:2 * G * d + H * dv].view(T, H, dv)
    decay = torch.exp(-torch.exp(a_log.double()) * pb.softplus(a.double() + bias.double()))[:, :, None].expand(T, H, d)
    want, S = plain_delta(q, k, v, pb.sigmoid(beta.double()), decay)
    for cuts in ([T], [1] * T, [7, 2, 1, 16, 17, 2]):
        got, state = walk("head_decay", qkv, beta, a, a_log, bias, H, G, d, dv, d ** -0.5, cuts)
        assert close(got.view(T, H, dv), want, 2e-5), cuts
        assert close(state, S, 2e-5), cuts


@pytest.mark.parametrize("H,d,dv,tau", [(2, 12, 20, 8.0), (4, 32, 32, 16.0), (1, 100, 7, 1.0), (3, 8, 6, 2.0), (2, 130, 64, 30.0)])
def test_gated_linear_attention_on_the_same_walk(H, d, dv, tau):
    g = torch.Generator().manual_seed(H * d + 1)
    T = 45
    qkv = torch.randn(T, 2 * H * d + H * dv + 4, generator=g)
    z, bias = torch.randn(T, H * d, generator=g) * 2, torch.randn(H * d, generator=g) + 1
    x = qkv.double()
    q, k = x[:, :H * d].view(T, H, d) * d ** -0.5, x[:, H * d:2 * H * d].view(T, H, d)
    v = x[:, 2 * H * d:2 * H * d + H * dv].view(T, H, dv)
    decay = (pb.sigmoid(z.double() + bias.double()) ** (1.0 / tau)).view(T, H, d)
    want, S = plain_delta(q, k, v, None, decay)
    for cuts, seg in (([T], 0), ([1] * T, 0), ([7, 2, 1, 16, 17, 2], 0), ([T], 16), ([T], 7), ([20, 25], 9), ([T], 44)):
        got, state = walk("sigmoid_decay", qkv, None, z, None, bias, H, H, d, dv, d ** -0.5, cuts, tau=tau,
                          segment_tokens=seg)
        assert close(got.view(T, H, dv), want, 2e-5), (cuts, seg)
        assert close(state, S, 2e-5), (cuts, seg)


@pytest.mark.parametrize("form", ["head_decay", "sigmoid_decay"])
def test_a_far_write_is_read_back_after_hundreds_of_tokens(form):
    """One token writes a value under a key of its own; 400 tokens later a query asks for that key.  In between the
    decays stay near one and the other keys are orthogonal to it, so what comes back is the value times the decay
    of 400 steps; a state that was lost or mixed up between the portions and single tokens gives something else."""
    H, d, dv, T, at = 2, 16, 8, 420, 11
    g = torch.Generator().manual_seed(5)
    key = torch.zeros(d); key[3] = 1.0
    others = torch.randn(T, H, d, generator=g); others[:, :, 3] = 0.0
    k = others.clone(); k[at] = key
    q = torch.randn(T, H, d, generator=g) * 0.01; q[:, :, 3] = 0.0; q[T - 1] = key * 5
    v = torch.randn(T, H, dv, generator=g)
    qkv = torch.cat([q.view(T, -1), k.view(T, -1), v.view(T, -1)], dim=1)
    if form == "head_decay":
        beta, a = torch.full((T, H), 9.0), torch.full((T, H), -6.0)      # write strength about one, decay near one
        a_log, bias = torch.zeros(H), torch.zeros(H)
        x = qkv.double()
        qq, kk = x[:, :H * d].view(T, H, d), x[:, H * d:2 * H * d].view(T, H, d)
        qq = qq / torch.sqrt((qq * qq).sum(-1, keepdim=True) + 1e-6)
        kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + 1e-6)
        decay = torch.exp(-pb.softplus(a.double()))[:, :, None].expand(T, H, d)
        want, _ = plain_delta(qq, kk, v.double(), pb.sigmoid(beta.double()), decay)
        args = (beta, a, a_log, bias)
        scale, tau = 1.0, 1.0
    else:
        z, bias = torch.full((T, H * d), 6.0), torch.zeros(H * d)
        decay = (pb.sigmoid(z.double()) ** 0.5).view(T, H, d)
        want, _ = plain_delta(qkv.double()[:, :H * d].view(T, H, d), qkv.double()[:, H * d:2 * H * d].view(T, H, d),
                              v.double(), None, decay)
        args = (None, z, None, bias)
        scale, tau = 1.0, 2.0
    assert float(want[T - 1].abs().max()) > 0.3                    # the far value is what the last read-out is made of
    runs = [([T], 0), ([300] + [1] * 120, 0), ([5, 2, 200] + [1] * 100 + [113], 0)]
    if form == "sigmoid_decay":
        runs += [([T], 64), ([300] + [1] * 120, 32)]                 # long portions walked in segments side by side
    for cuts, seg in runs:
        got, _ = walk(form, qkv, args[0], args[1], args[2], args[3], H, H, d, dv, scale, cuts, tau=tau, segment_tokens=seg)
        assert close(got.view(T, H, dv)[T - 1], want[T - 1], 5e-5), (cuts, seg)
        assert close(got.view(T, H, dv), want, 5e-5), (cuts, seg)


def test_unequal_requests_walked_in_segments_side_by_side():
    """Gated linear attention of three requests in one step, one of a single token, one shorter than a segment and
    one of many segments, in slots that hold states from before."""
    H, d, dv, seg = 3, 24, 40, 32
    g = torch.Generator().manual_seed(8)
    lens = [1, 20, 150]
    T = sum(lens)
    qkv = torch.randn(T, 2 * H * d + H * dv, generator=g)
    a, bias = torch.randn(T, H * d, generator=g), torch.randn(H * d, generator=g) + 1
    state0 = torch.randn(4, H * d * dv, generator=g) * 0.3
    slots = [2, 0, 3]
    x = qkv.double()
    state = state0.clone().to(DEV)
    got = F().delta_scan(qkv.to(DEV), None, 0, a.to(DEV), 0, None, bias.to(DEV), state, 0, i32([0, 1, 21, T]), i32(slots),
                         H, H, d, dv, d ** -0.5, form="sigmoid_decay", tau=4.0, segments=-(-150 // seg),
                         segment_tokens=seg).cpu().view(T, H, dv)
    lo = 0
    for n, slot in zip(lens, slots):
        rows = x[lo:lo + n]
        q, k = rows[:, :H * d].view(n, H, d) * d ** -0.5, rows[:, H * d:2 * H * d].view(n, H, d)
        v = rows[:, 2 * H * d:].view(n, H, dv)
        decay = (pb.sigmoid(a[lo:lo + n].double() + bias.double()) ** 0.25).view(n, H, d)
        S = state0[slot].double().view(H, d, dv).clone()
        out = []
        for t in range(n):
            S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
            out.append(torch.einsum("hkv,hk->hv", S, q[t]))
        assert close(got[lo:lo + n], torch.stack(out), 3e-5), n
        assert close(state[slot].cpu().view(H, d, dv), S, 3e-5), n
        lo += n
    assert torch.equal(state[1].cpu(), state0[1])          # a slot of no request is left alone


@pytest.mark.parametrize("heads,dv", [(4, 10), (2, 64), (3, 33), (1, 128)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_the_gate_behind_it(heads, dv, dtype):
    g = torch.Generator().manual_seed(heads + dv)
    T = 9
    o, gate = torch.randn(T, heads * dv, generator=g) * 4, torch.randn(T, heads * dv + 6, generator=g)
    w = 1 + 0.2 * torch.randn(dv, generator=g)
    x = o.double().view(T, heads, dv)
    z = gate.double()[:, 2:2 + heads * dv]
    want = (x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w.double()).reshape(T, -1) * pb.silu(z)
    got = F().gated_group_rmsnorm(o.to(DEV), gate.to(DEV), 2, w.to(DEV), heads, False, 1e-5, dtype, silu_after=True)
    assert close(got, want, 3e-6 if dtype == torch.float32 else 8e-3)


# --------------------------------------------------------------------------- #
# windowed attention with logistic key weights that are not normalised
# --------------------------------------------------------------------------- #

def paged(k, v, page_size, num_pages, seed, dtype):
    T, G, d = k.shape
    n = -(-T // page_size)
    order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed))[:n].tolist()
    kc = torch.full((num_pages, G, page_size, d), 99.0)
    vc = torch.full((num_pages, G, page_size, v.shape[2]), 99.0)
    for t in range(T):
        kc[order[t // page_size], :, t % page_size] = k[t]
        vc[order[t // page_size], :, t % page_size] = v[t]
    return kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), order


def plain_attention(q, k, v, scale, bias, window):
    T, H, d = q.shape
    G = k.shape[1]
    pos = torch.arange(T)
    vis = (pos[None, :] <= pos[:, None]) & (pos[:, None] - pos[None, :] < window)
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale + float(bias[h])
        out[:, h] = torch.where(vis, pb.sigmoid(s), torch.zeros((), dtype=torch.float64)) @ v[:, h // (H // G)].double()
    return out


def run_attention(q, k, v, scale, bias, window, cuts, dtype=torch.float32, page_size=8, tensor_cores=False,
                  freed_behind_window=False):
    """The kernel over a hand-made paged cache, the sequence's queries cut into steps ``cuts``; with
    ``freed_behind_window`` the pages that every later query's window has passed are taken out of the table, as
    the cache manager gives them back."""
    T, H, d = q.shape
    e = v.shape[2]
    kc, vc, order = paged(k, v, page_size, 2 * (-(-T // page_size)) + 3, 5, dtype)
    outs, lo = [], 0
    for n in cuts:
        table = list(order) + [-1] * 4
        if freed_behind_window:
            for p in range(len(order)):
                if (p + 1) * page_size <= lo - window + 1:
                    table[p] = -1
        table = i32([table])
        qq = q[lo:lo + n].to(dtype).to(DEV).contiguous()
        if tensor_cores == "memory" and n > 1:
            got = F().prefill_attention_tc_logistic(qq, kc, vc, table, i32([0, n]), i32([lo + n]), n, window, scale,
                                                    bias.to(DEV))
        elif tensor_cores:
            if n == 1:
                splits = F().attention_mix_tc_splits(min(window, lo + 1))
                po = torch.empty(splits * H * e, device=DEV)
                pm = torch.empty(splits * H * 2, device=DEV)
                got = F().attention_mix_tc(qq, kc, vc, None, table, i32([0, 1]), i32([lo + 1]), 1, window, scale, 0.0,
                                           splits, po, pm, head_bias=bias.to(DEV))
            else:
                got = F().attention_mix_tc(qq, kc, vc, None, table, i32([0, n]), i32([lo + n]), n, window, scale, 0.0,
                                           head_bias=bias.to(DEV))
        else:
            got = F().attention_mix(qq, kc, vc, None, table, i32([0, n]), i32([lo + n]), n, window, scale, 0.0,
                                    head_bias=bias.to(DEV))
        outs.append(got.cpu())
        lo += n
    assert lo == T
    return torch.cat(outs)


@pytest.mark.parametrize("H,G,d,e,window", [(4, 2, 16, 8, 9), (6, 3, 24, 40, 33), (1, 1, 20, 96, 1), (5, 1, 8, 8, 200),
                                            (2, 2, 64, 128, 70)])
def test_logistic_key_weights_against_plain_in_any_cut(H, G, d, e, window):
    g = torch.Generator().manual_seed(H + d)
    T = 83
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, e, generator=g)
    bias = torch.randn(H, generator=g)
    want = plain_attention(q, k, v, 0.3, bias, window)
    for cuts in ([T], [40] + [1] * 43, [7, 2, 13, 3, 2, 5, 17, 2, 31, 1]):
        got = run_attention(q, k, v, 0.3, bias, window, cuts, freed_behind_window=True)
        assert close(got, want, 3e-6), cuts


@pytest.mark.parametrize("H,G,d,e,window", [(4, 2, 32, 64, 21), (2, 1, 48, 128, 70), (10, 2, 16, 64, 5), (36, 2, 16, 64, 130),
                                            (4, 2, 64, 128, 136)])
def test_logistic_key_weights_on_the_tensor_cores(H, G, d, e, window):
    g = torch.Generator().manual_seed(H + d)
    T = 300
    r = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).float()
    q, k, v = r(T, H, d), r(T, G, d), r(T, G, e)
    bias = torch.randn(H, generator=g) - 1
    want = plain_attention(q, k, v, 0.2, bias, window)
    for cuts in ([T], [250] + [1] * 50, [7, 2, 130, 3, 2, 5, 17, 2, 131, 1]):
        got = run_attention(q, k, v, 0.2, bias, window, cuts, dtype=torch.bfloat16, tensor_cores=True,
                            freed_behind_window=True)
        assert close(got, want, 1.5e-2), cuts


@pytest.mark.parametrize("H,G,d,e,window", [(4, 2, 64, 128, 70), (2, 1, 128, 128, 300), (6, 3, 64, 64, 5), (4, 4, 128, 64, 129),
                                            (3, 1, 64, 128, 64)])
@pytest.mark.parametrize("page_size", [8, 16, 64])
def test_logistic_key_weights_on_the_tensor_memory_attention(H, G, d, e, window, page_size):
    """Prompt portions on the tcgen05 kernel (single tokens between them on the split kernel), portions that start
    inside key tiles and pages, with the pages behind the window given back."""
    g = torch.Generator().manual_seed(H + d + e)
    T = 400
    r = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).float()
    q, k, v = r(T, H, d), r(T, G, d), r(T, G, e)
    bias = torch.randn(H, generator=g) - 1
    want = plain_attention(q, k, v, 0.1, bias, window)
    for cuts in ([T], [250, 1, 1, 148], [7, 2, 130, 3, 2, 5, 17, 2, 131, 101]):
        got = run_attention(q, k, v, 0.1, bias, window, cuts, dtype=torch.bfloat16, tensor_cores="memory",
                            page_size=page_size, freed_behind_window=True)
        assert close(got, want, 1.5e-2), cuts
    F().check_tc_status()


@pytest.mark.parametrize("tensor_cores", [False, True, "memory"])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("window", [1, 2, 8, 9, 63, 64, 65, 136, 257])
def test_a_key_that_stands_out_just_inside_and_just_outside_the_window(window, decoded, tensor_cores):
    """The head's bias pushes every ordinary key's weight to nothing; one key carries a score that brings its own
    weight to one.  The last query must put out that key's value while the key is among the last ``window``
    positions, and nothing once it is one position further back."""
    H, G, d, e = 4, 2, 64, 64
    dtype = torch.bfloat16 if tensor_cores else torch.float32
    g = torch.Generator().manual_seed(window)
    T = 300
    for back in (window - 1, window, 0):                 # just inside, just outside, the query's own position
        key = T - 1 - back
        if key < 0:
            continue
        q = torch.randn(T, H, d, generator=g).to(torch.bfloat16).float() * 0.1
        k = torch.randn(T, G, d, generator=g).to(torch.bfloat16).float() * 0.1
        v = torch.randn(T, G, e, generator=g).to(torch.bfloat16).float()
        q[T - 1] = 0.0; q[T - 1, :, 0] = 8.0
        k[key] = 0.0; k[key, :, 0] = 8.0                  # score 64 * 0.5 = 32 against a bias of -16
        bias = torch.full((H,), -16.0)
        cuts = [T - 40] + [1] * 40 if decoded else [T - 37, 37]
        got = run_attention(q, k, v, 0.5, bias, window, cuts, dtype=dtype, tensor_cores=tensor_cores,
                            freed_behind_window=True)[T - 1].double()
        want = v[key].double().repeat_interleave(H // G, dim=0) if back < window else torch.zeros(H, e, dtype=torch.float64)
        assert float((got - want).abs().max()) <= 2e-2, (back, window)
        assert close(got, plain_attention(q, k, v, 0.5, bias, window)[T - 1], 1e-2) or back >= window


def test_the_first_tokens_of_a_sequence():
    H, G, d, e = 3, 1, 12, 10
    g = torch.Generator().manual_seed(2)
    q, k, v = torch.randn(5, H, d, generator=g), torch.randn(5, G, d, generator=g), torch.randn(5, G, e, generator=g)
    bias = torch.randn(H, generator=g)
    want = plain_attention(q, k, v, 0.3, bias, 3)
    for cuts in ([5], [1, 1, 1, 1, 1], [1, 4], [2, 3]):
        assert close(run_attention(q, k, v, 0.3, bias, 3, cuts), want, 3e-6), cuts
    # one token alone: its weight is the logistic function of its own score, not one
    one = run_attention(q[:1], k[:1], v[:1], 0.3, bias, 3, [1])[0].double()
    s = pb.sigmoid((q[0].double() @ k[0, 0].double()) * 0.3 + bias.double())
    assert float((one - s[:, None] * v[0, 0].double()[None, :]).abs().max()) < 1e-5


# --------------------------------------------------------------------------- #
# experts chosen within the best groups
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("T", [1, 5, 40, 300])
@pytest.mark.parametrize("E,K,count,keep", [(6, 2, 3, 2), (16, 4, 4, 3), (12, 5, 6, 3), (9, 2, 3, 1), (8, 3, 1, 1), (4, 4, 2, 2),
                                            (64, 6, 8, 2), (40, 1, 40, 7)])
def test_experts_chosen_within_the_best_groups_in_both_routings(T, E, K, count, keep):
    g = torch.Generator().manual_seed(T + E)
    W = 48
    x, wr = torch.randn(T, W, generator=g), torch.randn(E, W, generator=g) * 0.4
    want_idx, s = pb.route(x.double(), wr.double(), {"experts": E, "top": K, "groups": {"count": count, "keep": keep}})
    routers = [lambda: F().moe_router(x.to(DEV), wr.to(DEV), None, K, False, want_probs=True, groups=(count, keep))[:4]]
    if T <= F().route_small_max_tokens():
        ticket = torch.zeros(1 + T, dtype=torch.int32, device=DEV)
        routers.append(lambda: F().moe_route_small(x.to(DEV), wr.to(DEV), None, K, False, ticket, want_probs=True,
                                                   permute=False, groups=(count, keep))[:4])
    for route in routers:
        idx, w, _, probs = route()
        assert close(probs, s, 2e-6)
        assert sorted(map(sorted, idx.cpu().tolist())) == sorted(map(sorted, want_idx.tolist())) or \
            [sorted(r) for r in idx.cpu().tolist()] == [sorted(r) for r in want_idx.tolist()]
        assert [sorted(r) for r in idx.cpu().tolist()] == [sorted(r) for r in want_idx.tolist()]
        assert close(w, s.gather(1, idx.cpu().long()), 2e-6)            # the scores as they are
