"""The kernels that Nipapel added or widened, each against the plain function of the same mechanism (float64 on
the CPU), on sizes the tiny models do not reach, cut into portions and decoded, over hand-made paged caches,
with inputs made so that one key stands out just inside and just outside a window and the kept first keys."""

import pytest
import torch

import plain_nipapel as pn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def F():
    from mini_infer_b200.ops import functional
    return functional


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# --------------------------------------------------------------------------- #
# attention behind a window that keeps the first keys
# --------------------------------------------------------------------------- #

def paged(k, v, page_size, num_pages, seed, dtype, drop=()):
    """Scatter ``k [T, G, d]`` and ``v [T, G, e]`` over pages in a shuffled order; the logical pages in ``drop``
    are given back (their table entries are -1 and their memory holds other numbers)."""
    T, G, d = k.shape
    e = v.shape[2]
    n = -(-T // page_size)
    order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed))[:n].tolist()
    kc = torch.full((num_pages, G, page_size, d), 99.0)
    vc = torch.full((num_pages, G, page_size, e), 99.0)
    for t in range(T):
        if t // page_size in drop:
            continue
        kc[order[t // page_size], :, t % page_size] = k[t]
        vc[order[t // page_size], :, t % page_size] = v[t]
    table = [(-1 if i in drop else p) for i, p in enumerate(order)]
    return kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), table


def run_attention(q, k, v, window, keep, scale, cuts, dtype=torch.float32, page_size=8, tensor_cores=False,
                  release=False):
    """The kernel over a hand-made paged cache, the sequence's queries cut into steps ``cuts``.  ``release``:
    the first step has run already; only the later ones run (and are returned), over a cache whose pages
    between the kept first keys and the window of the first remaining query have been given back."""
    T, H, d = q.shape
    e = v.shape[2]
    drop, lo = (), 0
    if release:
        lo, cuts = cuts[0], cuts[1:]
        if window:
            drop = set(range(-(-keep // page_size), max(0, lo - window + 1) // page_size))
    kc, vc, table = paged(k, v, page_size, 2 * (-(-T // page_size)) + 3, 5, dtype, drop)
    table = i32([table + [-1] * 4])
    outs = []
    for n in cuts:
        qq = q[lo:lo + n].to(dtype).to(DEV).contiguous()
        if tensor_cores:
            kw = {}
            if n == 1:
                span = min(window, lo + 1) if window else lo + 1
                splits = F().attention_mix_tc_splits(span, keep)
                kw = dict(splits=splits, part_o=torch.full((splits * H * e,), 7.0, device=DEV),
                          part_ml=torch.full((splits * H * 2,), 7.0, device=DEV))
            got = F().attention_mix_tc(qq, kc, vc, None, table, i32([0, n]), i32([lo + n]), n, window, scale, 0.0,
                                       keep_first=keep, **kw)
        else:
            got = F().attention_mix(qq, kc, vc, None, table, i32([0, n]), i32([lo + n]), n, window, scale, 0.0,
                                    keep_first=keep)
        outs.append(got.float().cpu())
        lo += n
    return torch.cat(outs)


def plain_attention(q, k, v, window, keep, scale):
    T = q.shape[0]
    return pn.masked_softmax_attention(q.double(), k.double(), v.double(), scale, pn.visible(T, window or T, keep))


@pytest.mark.parametrize("H,G,d,e,window,keep", [(4, 2, 16, 8, 9, 3), (6, 3, 24, 40, 64, 1), (1, 1, 20, 96, 1, 1),
                                                 (5, 1, 8, 8, 17, 40), (16, 4, 64, 128, 40, 4), (3, 3, 130, 200, 23, 9),
                                                 (2, 2, 12, 12, 5, 0), (2, 1, 12, 12, 0, 6)])
def test_attention_with_kept_first_keys_against_plain_in_any_cut(H, G, d, e, window, keep):
    T = 75
    g = torch.Generator().manual_seed(H * 10 + d)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, e, generator=g)
    want = plain_attention(q, k, v, window, keep, 0.2)
    whole = run_attention(q, k, v, window, keep, 0.2, [T])
    assert float((whole.double() - want).abs().max()) <= 2e-5 * float(want.abs().max())
    for cuts in ([1] * T, [3, 2, 17, 1, 1, 33, 2, 16]):
        assert torch.equal(run_attention(q, k, v, window, keep, 0.2, cuts), whole)      # no bit moves
    # pages between the kept first keys and the window given back
    got = run_attention(q, k, v, window, keep, 0.2, [60, 2, 13], release=True)
    assert torch.equal(got, whole[60:])
    qb, kb, vb = (t.to(torch.bfloat16).float() for t in (q, k, v))
    want = plain_attention(qb, kb, vb, window, keep, 0.2)
    got = run_attention(qb, kb, vb, window, keep, 0.2, [T - 1, 1], torch.bfloat16)
    assert float((got.double() - want).abs().max()) <= 1e-2 * float(want.abs().max())


def stand_out(T, H, G, d, e, key, seed, bf16=False):
    """Queries and keys of which one key matches the last query a thousand times better than all others."""
    g = torch.Generator().manual_seed(seed)
    v = torch.randn(T, G, e, generator=g)
    k = torch.randn(T, G, d, generator=g) * 0.01
    q = torch.zeros(T, H, d)
    q[-1, :, 0] = 40.0
    k[key, :, 0] = 1.0
    if bf16:
        v, k = v.to(torch.bfloat16).float(), k.to(torch.bfloat16).float()
    return q, k, v


@pytest.mark.parametrize("window,keep", [(1, 1), (2, 5), (8, 8), (9, 7), (31, 9), (32, 1), (33, 16), (64, 17), (200, 3)])
@pytest.mark.parametrize("decoded", [False, True])
def test_a_key_that_stands_out_at_the_edges(window, keep, decoded):
    """Just inside the window, or among the kept first keys, the output is the key's value; just outside either
    it plays no part.  The same in a prompt's portion and decoded alone, with keys at page and tile borders and
    the pages in between given back."""
    T, H, G, d, e = 260, 2, 1, 8, 4
    cuts = [T - 1, 1] if decoded else [T - 5, 5]
    for key in (T - window, T - 1 - window, keep - 1, keep, 0):
        seen = key >= T - window or key < keep
        q, k, v = stand_out(T, H, G, d, e, key, window * 100 + keep)
        got = run_attention(q, k, v, window, keep, 1.0, cuts, release=True)[-1]
        hit = torch.allclose(got, v[key, 0].expand(H, e), atol=1e-4)
        assert hit == seen, (window, keep, key, decoded)
        want = plain_attention(q, k, v, window, keep, 1.0)[-1]
        assert torch.allclose(got.double(), want, atol=1e-5)


@pytest.mark.parametrize("H,G,d,e,window,keep", [(16, 4, 64, 128, 40, 4), (8, 2, 128, 128, 300, 1), (4, 2, 16, 64, 9, 20),
                                                 (24, 8, 32, 64, 64, 70), (5, 1, 48, 64, 17, 3), (40, 8, 32, 64, 33, 2)])
def test_kept_first_keys_on_the_tensor_cores(H, G, d, e, window, keep):
    assert F().attention_mix_tc_supported(H, G, d, e)
    T = 330
    g = torch.Generator().manual_seed(H + d)
    q, k, v = (torch.randn(T, n, s, generator=g).to(torch.bfloat16).float() for n, s in ((H, d), (G, d), (G, e)))
    want = plain_attention(q, k, v, window, keep, d ** -0.5)
    tol = 1.5e-2 * float(want.abs().max())
    for cuts in ([T], [200, 17, 3, 100] + [1] * 10, [310] + [1] * 20):
        got = run_attention(q, k, v, window, keep, d ** -0.5, cuts, torch.bfloat16, tensor_cores=True)
        assert float((got.double() - want).abs().max()) <= tol, cuts[:2]


@pytest.mark.parametrize("window,keep", [(1, 1), (15, 2), (16, 16), (17, 33), (128, 5), (129, 64), (257, 1)])
@pytest.mark.parametrize("decoded", [False, True])
def test_the_edges_on_the_tensor_cores(window, keep, decoded):
    T, H, G, d, e = 300, 4, 2, 16, 64
    cuts = [T - 1, 1] if decoded else [T - 7, 7]
    for key in (T - window, T - 1 - window, keep - 1, keep):
        seen = key >= T - window or key < keep
        q, k, v = stand_out(T, H, G, d, e, key, window + keep, bf16=True)
        got = run_attention(q, k, v, window, keep, 1.0, cuts, torch.bfloat16, tensor_cores=True, release=True)[-1]
        hit = torch.allclose(got, v[key].repeat_interleave(2, 0), atol=2e-2)
        assert hit == seen, (window, keep, key, decoded)


def test_a_far_kept_key_among_hundreds():
    T, H, G, d, e = 700, 4, 2, 16, 16
    q, k, v = stand_out(T, H, G, d, e, 2, 3)
    got = run_attention(q, k, v, 64, 3, 1.0, [T - 1, 1], page_size=16, release=True)[-1]
    assert torch.allclose(got, v[2].repeat_interleave(2, 0), atol=1e-4)
    q, k, v = stand_out(T, H, G, d, e, 3, 3)
    got = run_attention(q, k, v, 64, 3, 1.0, [T - 1, 1], page_size=16, release=True)[-1]
    assert not torch.allclose(got, v[3].repeat_interleave(2, 0), atol=1e-1)


# --------------------------------------------------------------------------- #
# head norms, rotation by halves, cache write
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dk,dv,rot", [(4, 2, 16, 8, 8), (3, 3, 40, 40, 40), (1, 1, 6, 10, 0), (5, 1, 130, 64, 2),
                                              (2, 1, 256, 128, 128), (9, 3, 48, 16, 12), (2, 2, 384, 64, 384)])
def test_head_norms_rotation_and_cache_write(dtype, nh, nkv, dk, dv, rot):
    T, ps, eps = 21, 4, 1e-5
    g = torch.Generator().manual_seed(nh + dk)
    qkv = torch.randn(T, (nh + nkv) * dk + nkv * dv, generator=g) * 3
    qg, kg = 1.0 + 0.3 * torch.randn(dk, generator=g), 1.0 + 0.3 * torch.randn(dk, generator=g)
    inv = torch.pow(torch.tensor(500.0, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1))
    pos = torch.arange(7, 7 + T)
    slots = torch.randperm(8 * ps, generator=g)[:T]
    slots[5] = -1
    kc = torch.zeros(8, nkv, ps, dk, dtype=dtype, device=DEV)
    vc = torch.zeros(8, nkv, ps, dv, dtype=dtype, device=DEV)
    q = F().rope_store(qkv.to(DEV), i32(pos.tolist()), inv.float().to(DEV) if rot else None, rot, i32(slots.tolist()), kc, vc,
                       nh, nkv, dk, dv, ps, dtype, qg.to(DEV), kg.to(DEV), eps).float().cpu()
    x = qkv.double()
    qq = pn.norm_plain(x[:, :nh * dk].view(T, nh, dk), qg.double(), eps)
    kk = pn.norm_plain(x[:, nh * dk:(nh + nkv) * dk].view(T, nkv, dk), kg.double(), eps)
    vv = x[:, (nh + nkv) * dk:].view(T, nkv, dv)
    if rot:
        # positions start at 7: rotate a longer sequence and take its tail
        pad = lambda t: torch.cat([torch.zeros(7, *t.shape[1:], dtype=t.dtype), t])
        qq, kk = pn.rotate_halves(pad(qq), rot, 500.0)[7:], pn.rotate_halves(pad(kk), rot, 500.0)[7:]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((q.double() - qq).abs().max()) <= tol * float(qq.abs().max())
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        assert float((kc[s // ps, :, s % ps].float().cpu().double() - kk[t]).abs().max()) <= tol * float(kk.abs().max())
        assert float((vc[s // ps, :, s % ps].float().cpu().double() - vv[t]).abs().max()) <= tol * float(vv.abs().max())
    assert int((kc != 0).any(dim=-1).sum()) == (T - 1) * nkv          # the row of slot -1 was written nowhere


# --------------------------------------------------------------------------- #
# attention through a latent: cached rows, queries, values as the leading part of the keys, gate
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,r,c", [(3, 8, 4, 20), (1, 20, 8, 24), (8, 32, 32, 128), (4, 4, 2, 10)])
def test_cached_rows_and_queries_of_the_latent_attention(dtype, H, d, r, c):
    T, ps, eps, base = 17, 4, 1e-6, 50.0
    g = torch.Generator().manual_seed(H + c)
    src = torch.randn(T, 5 + c + r + 3, generator=g) * 2
    gain = 1.0 + 0.2 * torch.randn(c, generator=g)
    inv = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * torch.arange(r // 2, dtype=torch.float64) / r).float()
    slots = torch.randperm(6 * ps, generator=g)[:T]
    slots[3] = -1
    cache = torch.zeros(6, 1, ps, c + r, dtype=dtype, device=DEV)
    F().latent_store(src.to(DEV), 5, i32(list(range(T))), inv.to(DEV), gain.to(DEV), eps, i32(slots.tolist()), cache, c, r)
    x = src.double()[:, 5:5 + c + r]
    lat = pn.norm_plain(x[:, :c], gain.double(), eps)
    kr = pn.rotate_neighbours(x[:, c:].reshape(T, 1, r), r, base).reshape(T, r)
    want = torch.cat([lat, kr], dim=1)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for t in range(T):
        s = int(slots[t])
        if s >= 0:
            got = cache[s // ps, 0, s % ps].float().cpu().double()
            assert float((got - want[t]).abs().max()) <= tol * float(want.abs().max()), t
    assert int((cache != 0).any(dim=-1).sum()) == T - 1
    q = torch.randn(T, H * (d + r), generator=g)
    q_full, q_plain = F().latent_query(q.to(DEV), i32(list(range(T))), inv.to(DEV), H, d, r, c, dtype, True)
    qq = q.double().view(T, H, d + r)
    rot = pn.rotate_neighbours(qq[..., d:], r, base)
    assert float((q_full[..., c:].float().cpu().double() - rot).abs().max()) <= tol * float(rot.abs().max())
    assert float((q_plain.float().cpu().double() - qq[..., :d]).abs().max()) <= tol * float(qq.abs().max())


@pytest.mark.parametrize("H,c,r,window,tc", [(3, 20, 4, 7, False), (5, 24, 8, 64, False), (4, 64, 16, 24, True),
                                             (8, 128, 32, 17, True), (1, 8, 2, 0, False)])
def test_values_that_are_the_leading_part_of_their_keys(H, c, r, window, tc):
    """One shared key/value head whose values are the first ``c`` numbers of the cached key rows."""
    T, ps = 150, 8
    dtype = torch.bfloat16 if tc else torch.float32
    g = torch.Generator().manual_seed(c + r)
    rows = torch.randn(T, 1, c + r, generator=g).to(dtype).float()
    q = (torch.randn(T, H, c + r, generator=g) * 0.5).to(dtype).float()
    want = pn.masked_softmax_attention(q.double(), rows.double(), rows.double()[..., :c], 0.3, pn.visible(T, window or T))
    cache, _, table = paged(rows, rows, ps, 2 * (-(-T // ps)) + 3, 9, dtype)
    table = i32([table])
    outs, lo = [], 0
    for n in [100, 2, 47, 1]:
        qq = q[lo:lo + n].to(dtype).to(DEV).contiguous()
        args = (qq, cache, cache, None, table, i32([0, n]), i32([lo + n]), n, window, 0.3, 0.0)
        if tc:
            assert F().attention_mix_tc_supported(H, 1, c + r, c)
            kw = {}
            if n == 1:
                splits = F().attention_mix_tc_splits(min(window, lo + 1) if window else lo + 1)
                kw = dict(splits=splits, part_o=torch.zeros(splits * H * c, device=DEV), part_ml=torch.zeros(splits * H * 2, device=DEV))
            outs.append(F().attention_mix_tc(*args, value_dim=c, **kw).float().cpu())
        else:
            outs.append(F().attention_mix(*args, value_dim=c).float().cpu())
        lo += n
    got = torch.cat(outs)
    assert got.shape == (T, H, c)
    assert float((got.double() - want).abs().max()) <= (1.5e-2 if tc else 2e-5) * float(want.abs().max())


def test_products_per_head_and_the_gate():
    T, H, K, N = 37, 5, 24, 12
    g = torch.Generator().manual_seed(0)
    x = torch.randn(T, 3 + H * (K + 2), generator=g)
    w = torch.randn(H, N, K, generator=g)
    out = torch.full((T, H * (N + 1) + 2), 5.0, device=DEV)
    F().dense_f32_heads(x.to(DEV), w.to(DEV), out=out, x_col=3, x_head_stride=K + 2, out_col=2, out_head_stride=N + 1)
    xs = torch.stack([x[:, 3 + h * (K + 2):3 + h * (K + 2) + K] for h in range(H)], 1).double()
    want = torch.einsum("thk,hnk->thn", xs, w.double())
    got = torch.stack([out[:, 2 + h * (N + 1):2 + h * (N + 1) + N] for h in range(H)], 1).cpu().double()
    assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
    assert float(out[:, :2].min()) == 5.0 and float(out[:, 2 + N].min()) == 5.0        # nothing beside the heads
    # the same rows alone or among others: no bit moves
    one = F().dense_f32_heads(x[5:6].contiguous().to(DEV), w.to(DEV), x_col=3, x_head_stride=K + 2)
    many = F().dense_f32_heads(x.to(DEV), w.to(DEV), x_col=3, x_head_stride=K + 2)
    assert torch.equal(one[0], many[5])
    a = torch.randn(T, H, N, generator=g)
    gate = torch.randn(T, 4 + H * N, generator=g)
    want = (a.double() * torch.sigmoid(gate.double()[:, 4:].view(T, H, N))).reshape(T, H * N)
    got = F().sigmoid_gate(a.to(DEV), False, gate.to(DEV), 4, H, N).cpu().double()
    assert torch.allclose(got, want, atol=1e-6)
    got = F().sigmoid_gate(a.transpose(0, 1).contiguous().to(DEV), True, gate.to(DEV), 4, H, N).cpu().double()
    assert torch.allclose(got, want, atol=1e-6)


# --------------------------------------------------------------------------- #
# feed-forward: bounded gated units, a router with a bias
# --------------------------------------------------------------------------- #

def test_bounded_gated_units():
    g = torch.Generator().manual_seed(1)
    gu = torch.randn(33, 2 * 50, generator=g) * 4
    for limit in (0.5, 2.0, 7.0):
        want = pn.clamped_glu(gu.double()[:, :50], gu.double()[:, 50:], limit)
        got = F().clamped_glu(gu.to(DEV), limit, 1.702, torch.float32).cpu().double()
        assert torch.allclose(got, want, atol=2e-6)
        assert float(got.max()) <= limit * (limit + 1.0) + 1e-6
    got = F().clamped_glu(gu.to(DEV), 2.0, 1.702, torch.bfloat16).float().cpu().double()
    assert torch.allclose(got, pn.clamped_glu(gu.double()[:, :50], gu.double()[:, 50:], 2.0), atol=3e-2)


@pytest.mark.parametrize("T", [1, 7, 40, 300])
@pytest.mark.parametrize("E,K", [(5, 2), (8, 3), (4, 4), (1, 1), (70, 6)])
def test_a_router_with_a_bias(T, E, K):
    H = 96
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, H, generator=g)
    wr = torch.randn(E, H, generator=g) / H ** 0.5
    b = torch.randn(E, generator=g)
    z = x.double() @ wr.double().T + b.double()
    top = torch.topk(z, K, dim=1)
    want_w = torch.softmax(top.values, dim=1)
    ticket = torch.zeros(1 + 128, dtype=torch.int32, device=DEV)
    runs = [F().moe_router(x.to(DEV), wr.to(DEV), None, K, True, bias=b.to(DEV))[:2]]
    if T <= F().route_small_max_tokens():
        runs.append(F().moe_route_small(x.to(DEV), wr.to(DEV), None, K, True, ticket, permute=False, bias=b.to(DEV))[:2])
    for idx, w in runs:
        idx, w = idx.cpu().long(), w.cpu().double()
        order = torch.argsort(idx, dim=1)
        want_order = torch.argsort(top.indices, dim=1)
        assert torch.equal(idx.gather(1, order), top.indices.gather(1, want_order))
        assert torch.allclose(w.gather(1, order), want_w.gather(1, want_order), atol=1e-5)
    # the bias takes part in the choice
    big = torch.zeros(E)
    big[E - 1] = 100.0
    idx = F().moe_router(x.to(DEV), wr.to(DEV), None, K, True, bias=big.to(DEV))[0].cpu()
    assert bool((idx == E - 1).any(dim=1).all())


def test_norm_with_an_offset_gain_and_the_norm_of_the_embedding():
    from mini_infer_b200.config import PartSpec, part_class
    from mini_infer_b200.parts.base import Runtime, precision_from_name
    g = torch.Generator().manual_seed(2)
    V, W, eps = 30, 44, 1e-5
    table = torch.randn(V, W, generator=g).to(torch.bfloat16)
    off = (0.3 * torch.randn(W, generator=g)).to(torch.bfloat16)
    ids = [3, 29, 0, 3, 17]
    want = pn.norm_one_plus(table.double()[ids], off.double(), eps)
    for dtype in ("float32", "bfloat16"):
        rt = Runtime(precision_from_name(dtype), torch.device(DEV))
        norm = PartSpec("rmsnorm", {"size": W, "eps": eps, "tensor": "embed.norm", "one_plus": True})
        emb = part_class("embedding", "token_embedding")({"vocab_size": V, "hidden_size": W, "tensor": "embed", "norm": norm}, "")
        assert [d.name for d in emb.tensor_decls()] == ["embed", "embed.norm"]
        emb.load({"embed": table, "embed.norm": off}, rt)
        got = emb.forward(i32(ids))
        assert got.dtype == torch.float32                      # the residual stream stays 32-bit
        assert torch.allclose(got.cpu().double(), want, atol=1e-5)
        part = part_class("norm", "rmsnorm")(norm.params, "")
        part.load({"embed.norm": off}, rt)
        hidden = torch.randn(6, W, generator=g)
        delta = torch.randn(6, W, generator=g)
        h = hidden.clone().to(DEV)
        out = part.apply(h, delta.to(DEV)).float().cpu().double()
        ref = pn.norm_one_plus((hidden + delta).double(), off.double(), eps)
        assert torch.allclose(out, ref, atol=1e-5 if dtype == "float32" else 3e-2)
        assert torch.allclose(h.cpu(), hidden + delta)


@pytest.mark.parametrize("T,E,K,H,I", [(3, 6, 2, 64, 64), (12, 4, 3, 128, 192), (40, 8, 2, 64, 128), (300, 8, 3, 128, 64)])
def test_bounded_gated_units_inside_every_grouped_product(T, E, K, H, I):
    """The experts' first product with the bounded gated unit formed in its epilogue: the CUDA-core form in both
    precisions, the decode-sized forms (sorted rows and by pair) and the tcgen05 form, against a loop over the
    chosen experts."""
    limit, slope = 1.3, 1.702
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, 2 * I, H, generator=g) * 2.0 / H ** 0.5).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    want = torch.zeros(T * K, I, dtype=torch.float64)
    for t in range(T):
        for k in range(K):
            gu = w[int(idx[t, k])].double() @ x[t].double()
            want[t * K + k] = pn.clamped_glu(gu[:I], gu[I:], limit)
    assert float(want.abs().max()) > 0.9 * limit          # the bound is met
    offsets, sorted_token, inv_perm = F().moe_permute(idx.to(DEV), E)
    inv = inv_perm.cpu().long()
    xd, wd = x.to(DEV), w.to(DEV)
    got = F().grouped_gemm_plain(xd.float(), sorted_token, wd.float(), offsets, T * K, True, torch.float32,
                                 glu=(limit, slope)).cpu().double()[inv]
    assert float((got - want).abs().max()) <= 1e-5 * limit * (limit + 1)
    tol = 2e-2 * limit * (limit + 1)
    got = F().grouped_gemm_plain(xd, sorted_token, wd, offsets, T * K, True, torch.bfloat16, glu=(limit, slope))
    assert float((got.float().cpu().double()[inv] - want).abs().max()) <= tol
    got = F().grouped_gemm_skinny(xd, sorted_token, wd, offsets, T * K, True, glu=(limit, slope))
    assert float((got.float().cpu().double()[inv] - want).abs().max()) <= tol
    if T <= F().skinny_pairs_max_tokens():
        got = F().grouped_gemm_skinny_pairs(xd, idx.to(DEV), wd, True, glu=(limit, slope))
        assert float((got.float().cpu().double() - want).abs().max()) <= tol
    got = F().grouped_gemm_tc(F().gather_rows(xd, sorted_token), wd, offsets, True, glu=(limit, slope))
    F().check_tc_status()
    assert float((got.float().cpu().double()[inv] - want).abs().max()) <= tol
    # without a form the same calls give silu(gate) * up as before
    got = F().grouped_gemm_skinny(xd, sorted_token, wd, offsets, T * K, True).float().cpu().double()[inv]
    ref = torch.zeros_like(want)
    for t in range(T):
        for k in range(K):
            gu = w[int(idx[t, k])].double() @ x[t].double()
            ref[t * K + k] = gu[:I] * torch.sigmoid(gu[:I]) * gu[I:]
    assert float((got - ref).abs().max()) <= 2e-2 * float(ref.abs().max())


@pytest.mark.parametrize("H,G,d,window,keep,ps", [(4, 2, 64, 40, 4, 16), (8, 2, 128, 300, 1, 16), (6, 3, 64, 9, 70, 8),
                                                  (2, 1, 128, 64, 64, 32), (3, 3, 64, 130, 17, 64)])
def test_kept_first_keys_in_the_tensor_memory_attention(H, G, d, window, keep, ps):
    """The tcgen05 prefill kernel behind a window that keeps the first keys: whole, in portions that start at any
    place, with single tokens beside them, and with the pages between kept keys and window given back."""
    assert F().prefill_attention_tc_supported(d, ps)
    T = 700
    g = torch.Generator().manual_seed(H + d + keep)
    q, k, v = (torch.randn(T, n, d, generator=g).to(torch.bfloat16).float() for n in (H, G, G))
    want = plain_attention(q, k, v, window, keep, d ** -0.5)
    tol = 1.5e-2 * float(want.abs().max())
    for cuts, release in (([T], False), ([200, 317, 3, 1, 179], False), ([450, 129, 1, 120], True)):
        lo, drop = 0, ()
        if release:
            lo, cuts = cuts[0], cuts[1:]
            drop = set(range(-(-keep // ps), max(0, lo - window + 1) // ps))
        kc, vc, table = paged(k, v, ps, 2 * (-(-T // ps)) + 3, 5, torch.bfloat16, drop)
        table = i32([table + [-1] * 4])
        start = lo
        outs = []
        for n in cuts:
            qq = q[lo:lo + n].to(torch.bfloat16).to(DEV).contiguous()
            outs.append(F().prefill_attention_tc(qq, kc, vc, table, i32([0, n]), i32([lo + n]), n, window, d ** -0.5,
                                                 keep_first=keep).float().cpu())
            lo += n
        F().check_tc_status()
        got = torch.cat(outs)
        assert float((got.double() - want[start:]).abs().max()) <= tol, (cuts, release)
    # a key that stands out among the kept ones, far behind the window
    for key in (keep - 1, keep):
        q2, k2, v2 = stand_out(T, H, G, d, d, key, keep, bf16=True)
        kc, vc, table = paged(k2, v2, ps, 2 * (-(-T // ps)) + 3, 5, torch.bfloat16)
        got = F().prefill_attention_tc(q2[-5:].to(torch.bfloat16).to(DEV).contiguous(), kc, vc, i32([table]), i32([0, 5]),
                                       i32([T]), 5, window, 1.0, keep_first=keep).float().cpu()[-1]
        seen = key < keep or key >= T - window
        assert torch.allclose(got, v2[key].repeat_interleave(H // G, 0), atol=2e-2) == seen, key


@pytest.mark.parametrize("H,c,r,window,ps", [(4, 64, 16, 24, 8), (16, 128, 64, 300, 16), (8, 128, 32, 17, 16), (1, 64, 8, 0, 32),
                                             (32, 64, 64, 1000, 64), (2, 128, 128, 129, 8)])
def test_heads_that_share_one_key_value_head_in_the_tensor_memory_attention(H, c, r, window, ps):
    """(query, head) pairs as the rows of a query tile; values are the leading part of the key rows; key rows
    that end inside a 64-column half."""
    assert F().prefill_attention_tc_shared_supported(H, c + r, c, ps)
    assert not F().prefill_attention_tc_shared_supported(6, c + r, c, ps)
    T = 700
    g = torch.Generator().manual_seed(H + c + r)
    rows = torch.randn(T, 1, c + r, generator=g).to(torch.bfloat16).float()
    q = (torch.randn(T, H, c + r, generator=g) * 0.5).to(torch.bfloat16).float()
    scale = (c + r) ** -0.5
    want = pn.masked_softmax_attention(q.double(), rows.double(), rows.double()[..., :c], scale, pn.visible(T, window or T))
    tol = 1.5e-2 * float(want.abs().max())
    for cuts, release in (([T], False), ([200, 317, 3, 1, 179], False), ([450, 129, 1, 120], True)):
        lo, drop = 0, ()
        if release:
            lo, cuts = cuts[0], cuts[1:]
            if window:
                drop = set(range(0, max(0, lo - window + 1) // ps))
        cache, _, table = paged(rows, rows, ps, 2 * (-(-T // ps)) + 3, 9, torch.bfloat16, drop)
        table = i32([table + [-1] * 4])
        start, outs = lo, []
        for n in cuts:
            qq = q[lo:lo + n].to(torch.bfloat16).to(DEV).contiguous()
            outs.append(F().prefill_attention_tc_shared(qq, cache, table, i32([0, n]), i32([lo + n]), n, window, scale, c).float().cpu())
            lo += n
        F().check_tc_status()
        got = torch.cat(outs)
        assert got.shape == (T - start, H, c)
        assert float((got.double() - want[start:]).abs().max()) <= tol, (cuts, release)
    # two requests of unequal portions in one launch
    cache, _, table = paged(rows, rows, ps, 2 * (-(-T // ps)) + 3, 9, torch.bfloat16)
    qq = torch.cat([q[100:130], q[699:700]]).to(torch.bfloat16).to(DEV).contiguous()
    got = F().prefill_attention_tc_shared(qq, cache, i32([table, table]), i32([0, 30, 31]), i32([130, 700]), 30, window,
                                          scale, c).float().cpu().double()
    F().check_tc_status()
    assert float((got[:30] - want[100:130]).abs().max()) <= tol and float((got[30] - want[699]).abs().max()) <= tol
