"""The kernels and part options that Tofinex added, each against the plain function of the same mechanism
(float64 on the CPU), on sizes the tiny models do not reach, cut into portions and decoded, over hand-made paged
caches, with inputs made so that a fault shows: a key that stands out far back among hundreds, queries that match
no key (whose weight the added key of the softmax must take), the first token of a sequence."""

from types import SimpleNamespace

import pytest
import torch

import plain_tofinex as pt

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def F():
    from mini_infer_b200.ops import functional
    return functional


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def runtime(dtype):
    from mini_infer_b200.parts.base import Runtime, configure_matmul_exactness, precision_from_name
    configure_matmul_exactness()
    return Runtime(precision_from_name(dtype), torch.device(DEV))


# --------------------------------------------------------------------------- #
# head norms, rotation of neighbouring dimensions, blended values, cache write
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("H,G,d,e,rot,blend,pad", [
    (4, 2, 16, 10, 8, True, 5), (5, 1, 12, 20, 12, False, 5), (1, 1, 6, 3, 2, True, 5), (3, 3, 34, 34, 0, True, 5),
    (8, 2, 96, 64, 96, True, 5),
    # sizes in fours and rows on 16-byte boundaries (a warp per head): all of a head rotated, part of it, none;
    # heads of more than 128 and of more than 256 numbers; more heads than one block's eight warps
    (8, 2, 96, 64, 96, True, 8), (4, 2, 160, 48, 80, True, 4), (2, 1, 320, 132, 320, False, 0),
    (3, 1, 8, 4, 4, True, 12), (13, 13, 64, 64, 0, True, 8), (2, 2, 12, 12, 6, True, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norms_neighbour_rotation_and_blended_values_reach_the_cache(H, G, d, e, rot, blend, pad, dtype):
    T, first, ps = 21, 37, 8                  # the rows are positions 37 .. 57 of their request
    g = torch.Generator().manual_seed(H + d)
    qkv = torch.randn(T, (H + G) * d + G * e, generator=g)
    qg, kg = 1.0 + 0.3 * torch.randn(d, generator=g), 1.0 + 0.3 * torch.randn(d, generator=g)
    wide = torch.randn(T, G * e + pad, generator=g)         # the first layer's values lie inside wider rows
    lam = torch.tensor([0.3])
    base, eps = 300.0, 1e-5
    pages = 10
    slots = torch.randperm(pages * ps, generator=g)[:T].to(torch.int32)
    kc = torch.zeros(pages, G, ps, d, dtype=dtype, device=DEV)
    vc = torch.zeros(pages, G, ps, e, dtype=dtype, device=DEV)
    inv = None
    if rot:
        inv = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)
        inv = inv.float().to(DEV)
    vf = wide.to(DEV)[:, pad:] if blend else None
    q = F().rope_store(qkv.to(DEV), i32(list(range(first, first + T))), inv, rot, slots.to(DEV), kc, vc, H, G, d, e, ps,
                       dtype, qg.to(DEV), kg.to(DEV), eps, neighbours=True, v_first=vf,
                       blend=lam.to(DEV) if blend else None)
    x = qkv.double()
    wq = pt.norm_plain(x[:, :H * d].view(T, H, d), qg.double(), eps)
    wk = pt.norm_plain(x[:, H * d:(H + G) * d].view(T, G, d), kg.double(), eps)
    if rot:
        wq, wk = pt.rotate_neighbours(wq, rot, base, first), pt.rotate_neighbours(wk, rot, base, first)
    wv = x[:, (H + G) * d:].view(T, G, e)
    if blend:
        wv = pt.blend_values(wv, wide[:, pad:].double(), float(lam))
    tol = 5e-6 if dtype == torch.float32 else 8e-3       # float32 angles at positions up to 57
    assert float((q.double().cpu() - wq).abs().max()) <= tol * float(wq.abs().max())
    for t in range(T):
        page, off = int(slots[t]) // ps, int(slots[t]) % ps
        assert float((kc[page, :, off].double().cpu() - wk[t]).abs().max()) <= tol * float(wk.abs().max())
        assert float((vc[page, :, off].double().cpu() - wv[t]).abs().max()) <= tol * float(wv.abs().max())
    assert float(kc.float().abs().sum()) > 0 and int((kc.float().abs().sum(dim=(1, 3)) > 0).sum()) == T


# --------------------------------------------------------------------------- #
# attention with capped scores and a softmax that counts one key more
# --------------------------------------------------------------------------- #

def paged(k, v, page_size, num_pages, seed, dtype):
    T, G, d = k.shape
    e = v.shape[2]
    n = -(-T // page_size)
    order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed))[:n].tolist()
    kc = torch.full((num_pages, G, page_size, d), 99.0)
    vc = torch.full((num_pages, G, page_size, e), 99.0)
    for t in range(T):
        kc[order[t // page_size], :, t % page_size] = k[t]
        vc[order[t // page_size], :, t % page_size] = v[t]
    return kc.to(dtype).to(DEV), vc.to(dtype).to(DEV), order


def run_attention(q, k, v, scale, cap, cuts, dtype=torch.float32, page_size=8, tensor_cores=False, sink=True,
                  tensor_memory=False):
    """The kernel over a hand-made paged cache, the sequence's queries cut into steps ``cuts``."""
    T, H, d = q.shape
    e = v.shape[2]
    kc, vc, table = paged(k, v, page_size, 2 * (-(-T // page_size)) + 3, 5, dtype)
    table = i32([table + [-1] * 4])
    outs, lo = [], 0
    for n in cuts:
        qq = q[lo:lo + n].to(dtype).to(DEV).contiguous()
        if tensor_memory:
            got = F().prefill_attention_tc(qq, kc, vc, table, i32([0, n]), i32([lo + n]), n, 0, scale, softcap=cap,
                                           sink=sink)
            F().check_tc_status()
        elif tensor_cores:
            kw = {}
            if n == 1:
                splits = F().attention_mix_tc_splits(lo + 1, 0)
                kw = dict(splits=splits, part_o=torch.full((splits * H * e,), 7.0, device=DEV),
                          part_ml=torch.full((splits * H * 2,), 7.0, device=DEV))
            got = F().attention_mix_tc(qq, kc, vc, None, table, i32([0, n]), i32([lo + n]), n, 0, scale, cap,
                                       sink=sink, **kw)
        else:
            got = F().attention_mix(qq, kc, vc, None, table, i32([0, n]), i32([lo + n]), n, 0, scale, cap, sink=sink)
        outs.append(got.float().cpu())
        lo += n
    return torch.cat(outs)


def plain_attention(q, k, v, scale, cap):
    T, H, _ = q.shape
    G = k.shape[1]
    kk, vv = k.double().repeat_interleave(H // G, dim=1), v.double().repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q.double(), kk) * scale
    if cap:
        s = pt.cap(s, cap)
    pos = torch.arange(T)
    p = pt.sink_softmax(s, (pos[None, :] <= pos[:, None])[None].expand(H, T, T))
    return torch.einsum("hij,jhe->ihe", p, vv)


@pytest.mark.parametrize("H,G,d,e,cap", [(4, 2, 16, 8, 3.0), (6, 3, 24, 40, 0.0), (1, 1, 20, 96, 1.5), (5, 1, 8, 8, 7.0),
                                         (3, 3, 130, 200, 4.0), (8, 2, 96, 64, 20.0)])
def test_attention_with_one_key_more_against_plain_in_any_cut(H, G, d, e, cap):
    T = 75
    g = torch.Generator().manual_seed(H * 10 + d)
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, e, generator=g)
    want = plain_attention(q, k, v, 0.3, cap)
    whole = run_attention(q, k, v, 0.3, cap, [T])
    assert float((whole.double() - want).abs().max()) <= 2e-5 * float(want.abs().max())
    for cuts in ([1] * T, [3, 2, 17, 1, 1, 33, 2, 16]):
        assert torch.equal(run_attention(q, k, v, 0.3, cap, cuts), whole)      # no bit moves
    # without the added key the result differs: the comparison above would see a kernel that left it out
    assert float((run_attention(q, k, v, 0.3, cap, [T], sink=False).double() - want).abs().max()) > 1e-2
    qb, kb, vb = (t.to(torch.bfloat16).float() for t in (q, k, v))
    want = plain_attention(qb, kb, vb, 0.3, cap)
    got = run_attention(qb, kb, vb, 0.3, cap, [T - 1, 1], torch.bfloat16)
    assert float((got.double() - want).abs().max()) <= 1e-2 * float(want.abs().max())


@pytest.mark.parametrize("H,G,d,e", [(4, 2, 32, 64), (2, 2, 16, 64), (36, 2, 16, 64), (2, 1, 48, 128), (16, 4, 128, 128)])
def test_tensor_core_attention_with_one_key_more(H, G, d, e):
    """Prompt portions, and single tokens whose keys are split over blocks and merged (the added key is counted
    once, by the merge)."""
    assert F().attention_mix_tc_supported(H, G, d, e)
    T = 330
    g = torch.Generator().manual_seed(H + e)
    q, k, v = (torch.randn(T, n, s, generator=g).to(torch.bfloat16).float() for n, s in ((H, d), (G, d), (G, e)))
    want = plain_attention(q, k, v, 0.25, 5.0)
    for cuts in ([T], [200, 17, 2, 1, 1, 1, 100, 1, 1, 1, 1, 1, 1, 1, 1]):
        got = run_attention(q, k, v, 0.25, 5.0, cuts, torch.bfloat16, page_size=16, tensor_cores=True)
        assert float((got.double() - want).abs().max()) <= 1.2e-2 * float(want.abs().max())
    got = run_attention(q, k, v, 0.25, 5.0, [T - 1, 1], torch.bfloat16, page_size=16, tensor_cores=True, sink=False)
    assert float((got.double() - want).abs().max()) > 2e-2 * float(want.abs().max())


@pytest.mark.parametrize("H,G,d,cap", [(4, 2, 64, 5.0), (2, 2, 128, 30.0), (6, 1, 128, 0.0), (3, 3, 64, 1.0)])
def test_tensor_memory_attention_with_capped_scores_and_one_key_more(H, G, d, cap):
    """Prompt portions on the tcgen05 kernel: whole, and in portions that start inside key tiles and pages."""
    T = 450
    g = torch.Generator().manual_seed(H + d)
    q, k, v = (torch.randn(T, n, d, generator=g).to(torch.bfloat16).float() for n in (H, G, G))
    want = plain_attention(q, k, v, 0.15, cap)
    for cuts in ([T], [130, 2, 200, 17, 101]):
        got = run_attention(q, k, v, 0.15, cap, cuts, torch.bfloat16, page_size=16, tensor_memory=True)
        assert float((got.double() - want).abs().max()) <= 1.2e-2 * float(want.abs().max())
    got = run_attention(q, k, v, 0.15, cap, [T], torch.bfloat16, page_size=16, tensor_memory=True, sink=False)
    assert float((got.double() - want).abs().max()) > 2e-2 * float(want.abs().max())
    if cap:
        other = plain_attention(q, k, v, 0.15, 0.0)
        assert float((other - want).abs().max()) > 2e-2 * float(want.abs().max())      # the cap matters here


@pytest.mark.parametrize("H,G,d,cap,split", [(4, 2, 64, 5.0, 128), (2, 2, 128, 30.0, 512), (6, 1, 128, 0.0, 256),
                                             (3, 3, 64, 1.0, 512), (2, 1, 256, 8.0, 128)])
def test_split_attention_of_single_tokens_with_capped_scores_and_one_key_more(H, G, d, cap, split):
    """Two requests of unequal length decode side by side on the split-KV kernel: each against the plain
    attention of its last token, with splits that end inside pages; a query that matches nothing gives its
    weight to the added key."""
    g = torch.Generator().manual_seed(H + d)
    lens = [701, 130]
    seqs = [[torch.randn(T, n, d, generator=g).to(torch.bfloat16).float() for n in (H, G, G)] for T in lens]
    # the second request's last query stands against every one of its keys: scores as far below zero as the cap lets them
    seqs[1][1][:, :, 0] = 3.0
    seqs[1][0][-1] = 0.0
    seqs[1][0][-1, :, 0] = -20.0
    ps, pages = 16, 120
    kc = torch.full((pages, G, ps, d), 99.0)
    vc = torch.full((pages, G, ps, d), 99.0)
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.full((2, 50), -1, dtype=torch.int32)
    for b, (q, k, v) in enumerate(seqs):
        for t in range(lens[b]):
            if t % ps == 0:
                table[b, t // ps] = order.pop()
            kc[table[b, t // ps], :, t % ps], vc[table[b, t // ps], :, t % ps] = k[t], v[t]
    qq = torch.stack([s[0][-1] for s in seqs]).to(torch.bfloat16).to(DEV)
    splits = -(-max(lens) // split)
    po, pml = torch.full((2 * H * splits * d,), 7.0, device=DEV), torch.full((2 * H * splits * 2,), 7.0, device=DEV)
    for sink in (True, False):
        got = F().decode_attention(qq, kc.to(torch.bfloat16).to(DEV), vc.to(torch.bfloat16).to(DEV), table.to(DEV),
                                   i32([0, 1, 2]), i32(lens), po, pml, splits, 0, scale=0.15, split=split, softcap=cap,
                                   sink=sink).float().cpu()
        for b, (q, k, v) in enumerate(seqs):
            want = plain_attention(q, k, v, 0.15, cap)[-1]
            err = float((got[b].double() - want).abs().max()) / float(want.abs().max())
            if sink:
                assert err <= 1.2e-2, (b, err)
            elif b == 1 and (cap == 0.0 or cap >= 5.0):
                # (a cap of 1 holds every score above -1, and hundreds of such keys outweigh the added one)
                assert err > 2e-2, err      # the query that matches nothing: without the added key it must attend


@pytest.mark.parametrize("tensor_cores", [False, True, "memory"])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("key", [0, 1, 63, 64, 65, 255, 256, 500, 699])
def test_a_far_key_among_hundreds_and_queries_that_match_nothing(key, decoded, tensor_cores):
    """The last query matches one key a thousand times better than the others: its output is that key's value,
    wherever the key lies (the first tokens, page and tile borders, far back).  The query before it matches
    nothing, with scores far below zero: the added key takes all of its weight and its output is zero."""
    T, H, G, d, e = 700, 4, 2, 32, 64
    if tensor_cores == "memory":
        d = 64                                  # the tcgen05 kernel: keys and values of one size, portions only
        if decoded:
            pytest.skip("single tokens take the split kernel")
    g = torch.Generator().manual_seed(key)
    v = torch.randn(T, G, e, generator=g).to(torch.bfloat16).float()
    k = (torch.randn(T, G, d, generator=g) * 0.01).to(torch.bfloat16).float()
    k[:, :, 1] = 1.0
    q = torch.zeros(T, H, d)
    q[-1, :, 0] = 40.0
    k[key, :, 0] = 1.0
    q[-2, :, 1] = -30.0                         # every score of this query is -30 * scale
    dtype = torch.bfloat16 if tensor_cores else torch.float32
    cuts = [T - 2, 1, 1] if decoded else [T]
    got = run_attention(q, k, v, 1.0, 50.0, cuts, dtype, page_size=16, tensor_cores=tensor_cores is True,
                        tensor_memory=tensor_cores == "memory")
    want = plain_attention(q, k, v, 1.0, 50.0)
    tol = 1e-2 if tensor_cores else 1e-4
    assert float((got[-1].double() - v[key].double().repeat_interleave(H // G, dim=0)).abs().max()) <= tol
    assert float(got[-2].abs().max()) <= 1e-6
    assert float((got[-2:].double() - want[-2:]).abs().max()) <= tol


def test_the_first_token_shares_its_weight_with_the_added_key():
    """A sequence of one token: the weight of its own key is ``exp(s) / (1 + exp(s))``, not one."""
    H, G, d, e = 2, 1, 16, 8
    g = torch.Generator().manual_seed(1)
    q, k, v = torch.randn(1, H, d, generator=g), torch.randn(1, G, d, generator=g), torch.randn(1, G, e, generator=g)
    got = run_attention(q, k, v, 0.2, 0.0, [1])
    s = (q[0].double() @ k[0, 0].double()) * 0.2
    want = (torch.exp(s) / (1 + torch.exp(s)))[:, None] * v[0, 0].double()[None]
    assert float((got[0].double() - want).abs().max()) <= 1e-6


# --------------------------------------------------------------------------- #
# a part's output normalised and added to the residual
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("T,W", [(1, 40), (7, 192), (33, 1000), (3, 9000), (5, 1026), (4, 1536), (2, 4100), (2, 6000)])
@pytest.mark.parametrize("dtype", [None, torch.bfloat16])
def test_output_norm_and_scaled_addition(T, W, dtype):
    g = torch.Generator().manual_seed(T + W)
    hidden, y, w = torch.randn(T, W, generator=g), 3.0 * torch.randn(T, W, generator=g), 1 + 0.2 * torch.randn(W, generator=g)
    want = hidden.double() + 0.6 * pt.norm_plain(y.double(), w.double(), 1e-5)
    h = hidden.to(DEV).clone()
    x = F().out_norm_add(h, y.to(DEV), w.to(DEV), 1e-5, 0.6, dtype)
    assert float((h.double().cpu() - want).abs().max()) <= 2e-6 * float(want.abs().max())
    if dtype is None:
        assert x is None
    else:
        assert torch.equal(x, h.to(dtype))
    # a sum of rows formed inside the kernel: rows by index, weights or none, an extra term with its scale
    K, N = 3, T * 3
    rows, idx = torch.randn(N, W, generator=g), torch.randperm(N, generator=g).to(torch.int32).view(T, K)
    wk, extra, scale = torch.rand(T, K, generator=g), torch.randn(T, W, generator=g), torch.rand(T, generator=g)
    for use_w, use_extra, use_idx in ((True, True, True), (False, False, True), (False, True, False)):
        picked = rows[idx.long()] if use_idx else rows.view(T, K, W)
        s = (picked.double() * (wk.double()[:, :, None] if use_w else 1.0)).sum(dim=1)
        if use_extra:
            s = s + scale.double()[:, None] * extra.double()
        want = hidden.double() + 0.6 * pt.norm_plain(s, w.double(), 1e-5)
        h = hidden.to(DEV).clone()
        tup = (rows.to(DEV), idx.to(DEV) if use_idx else None,
               wk.to(DEV) if use_w else (None if use_idx else torch.ones(T, K, device=DEV)),
               extra.to(DEV) if use_extra else None, scale.to(DEV) if use_extra else None)
        F().out_norm_add(h, tup, w.to(DEV), 1e-5, 0.6, dtype)
        assert float((h.double().cpu() - want).abs().max()) <= 3e-6 * float(want.abs().max())


def test_capped_logits_and_rounded_rows():
    z = torch.randn(5, 333) * 40
    got = F().softcap_rows(z.to(DEV).clone(), 30.0)
    assert float((got.double().cpu() - pt.cap(z.double(), 30.0)).abs().max()) <= 1e-5
    assert torch.equal(F().cast_rows(z.to(DEV), torch.bfloat16).cpu(), z.to(torch.bfloat16))


# --------------------------------------------------------------------------- #
# a router that scores with the logistic function, weights on the experts' inputs
# --------------------------------------------------------------------------- #

@pytest.mark.parametrize("T", [1, 5, 40, 300])
@pytest.mark.parametrize("E,K", [(5, 2), (16, 1), (3, 3), (1, 1), (60, 4)])
def test_sigmoid_router_in_both_routings(T, E, K):
    W = 72
    g = torch.Generator().manual_seed(T + E)
    x, wr, wg = torch.randn(T, W, generator=g), torch.randn(E, W, generator=g) * 0.3, torch.randn(W, generator=g) * 0.3
    idx_w, w_w, scores = pt.router_choice(x.double(), wr.double(), K)
    calls = [lambda: F().moe_router(x.to(DEV), wr.to(DEV), wg.to(DEV), K, False, want_probs=True, scoring="sigmoid")]
    if T <= F().route_small_max_tokens():
        ticket = torch.zeros(1 + T, dtype=torch.int32, device=DEV)
        calls.append(lambda: F().moe_route_small(x.to(DEV), wr.to(DEV), wg.to(DEV), K, False, ticket, want_probs=True,
                                                 scoring="sigmoid")[:4])
    for call in calls:
        idx, w, gate, probs = call()
        assert float((probs.double().cpu() - scores).abs().max()) <= 1e-5
        assert float((gate.double().cpu() - torch.sigmoid(x.double() @ wg.double())).abs().max()) <= 1e-5
        same = (idx.cpu().long() == idx_w).all(dim=1)
        # a row that differs does so at a near-tie of the last chosen and the first left-out score
        s = torch.sort(scores, dim=1, descending=True).values
        if K < E:
            assert float((s[~same, K - 1] - s[~same, K]).abs().max() if (~same).any() else 0.0) <= 1e-5
        assert float((w.double().cpu() - scores.gather(1, idx.cpu().long())).abs().max()) <= 1e-5
        assert all(len(set(r)) == K for r in idx.cpu().tolist())


def test_numbers_brought_into_expert_order():
    g = torch.Generator().manual_seed(3)
    for n in (1, 27, 1000):
        v = torch.rand(n, generator=g)
        dest = torch.randperm(n, generator=g).to(torch.int32)
        got = F().scatter_values(v.to(DEV), dest.to(DEV)).cpu()
        want = torch.empty(n)
        want[dest.long()] = v
        assert torch.equal(got, want)


@pytest.mark.parametrize("form", ["plain32", "plain16", "skinny", "pairs", "pairs_large", "tc"])
def test_a_number_per_row_that_scales_both_halves_of_a_gated_unit(form):
    """Every grouped product's epilogue: ``silu(s g) (s u)`` with ``g``, ``u`` the products of the unscaled row,
    against the gated unit of the scaled row.  The scale matters: without it the result is far off."""
    g = torch.Generator().manual_seed(len(form))
    E, Kd, Nout = 5, 64, 96
    w = (torch.randn(E, 2 * Nout, Kd, generator=g) * Kd ** -0.5).to(torch.bfloat16)
    if form.startswith("pairs"):
        T, K = (6, 2) if form == "pairs" else (50, 3)
        x = torch.randn(T, Kd, generator=g).to(torch.bfloat16)
        idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
        scale = 0.1 + torch.rand(T, K, generator=g)
        rows, experts = x.repeat_interleave(K, dim=0), idx.reshape(-1).long()
        call = lambda sc: F().grouped_gemm_skinny_pairs(x.to(DEV), idx.to(DEV), w.to(DEV), True, row_scale=sc)
    else:
        counts = [37, 0, 1, 150 if form == "tc" else 9, 16]
        n = sum(counts)
        offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
        rows = torch.randn(n, Kd, generator=g).to(torch.bfloat16)
        experts = torch.repeat_interleave(torch.arange(E), torch.tensor(counts))
        scale = 0.1 + torch.rand(n, generator=g)
        dt = torch.float32 if form == "plain32" else torch.bfloat16
        a, wd, off = rows.to(dt).to(DEV), w.to(dt).to(DEV), offsets.to(DEV)
        if form.startswith("plain"):
            call = lambda sc: F().grouped_gemm_plain(a, None, wd, off, n, True, dt, row_scale=sc)
        elif form == "skinny":
            call = lambda sc: F().grouped_gemm_skinny(a, None, wd, off, n, True, row_scale=sc)
        else:
            def call(sc):
                out = F().grouped_gemm_tc(a, wd, off, True, row_scale=sc)
                F().check_tc_status()
                return out
    xs = rows.double() * scale.reshape(-1, 1).double()
    gu = torch.einsum("nk,nfk->nf", xs, w.double()[experts])
    want = torch.nn.functional.silu(gu[:, :Nout]) * gu[:, Nout:]
    got = call(scale.to(DEV)).double().cpu()
    tol = 1e-5 if form == "plain32" else 1.2e-2
    assert float((got - want).abs().max()) <= tol * float(want.abs().max())
    assert float((call(None).double().cpu() - want).abs().max()) > 0.1 * float(want.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [1, 6, 40, 700])
@pytest.mark.parametrize("W,E,K,ff,shared", [(64, 4, 2, 64, 64), (96, 16, 1, 96, 0), (72, 5, 5, 24, 40), (40, 1, 1, 16, 16)])
def test_expert_block_with_weights_on_the_inputs(dtype, T, W, E, K, ff, shared):
    """The whole part against the plain block, in every form its products take (a few rows per expert, the
    tensor-core tiles, the plain kernel) and as a pending sum that the block's norm kernel forms."""
    from mini_infer_b200.config import part_class
    rt = runtime(dtype)
    params = {"hidden_size": W, "num_experts": E, "top_k": K, "expert_intermediate_size": ff,
              "shared_intermediate_size": shared, "norm_topk_prob": False, "scoring": "sigmoid", "weight_input": True,
              "router": "router", "expert": "e{e}.", "gate": "gate", "up": "up", "down": "down", "shared": "shared.",
              "shared_gate": "shared.sg"}
    part = part_class("feed_forward", "sparse_moe")(params, "f.")
    g = torch.Generator().manual_seed(W + T)
    t = {d.name: (torch.randn(*d.shape, generator=g) * (2.0 / d.shape[-1] ** 0.5)).to(torch.bfloat16)
         for d in part.tensor_decls()}
    part.load(t, rt)
    part.keep_routing = True
    x = torch.randn(T, W, generator=g).to(torch.bfloat16)
    out = part.forward(x.to(rt.act).to(DEV), SimpleNamespace(prefetch=None))      # (a step without weight prefetch)
    idx = part.last_routing[0].cpu().long()
    mlp = {"router": {"top": K}, "shared": {"ff": shared} if shared else None}
    rnd = pt.same if dtype == "float32" else pt.as_bfloat16
    w64 = {k: v.double() for k, v in t.items()}
    ref, (ref_idx, scores) = pt.moe(x.double(), w64, "f.", mlp, rnd, forced=idx)
    kth = torch.sort(scores, dim=1, descending=True).values[:, K - 1]
    assert float((kth[:, None] - scores.gather(1, idx)).max()) <= (1e-5 if dtype == "float32" else 1e-3)
    tol = 3e-5 if dtype == "float32" else 2e-2
    assert float((out.double().cpu() - ref).abs().max()) <= tol * float(ref.abs().max())
    # the experts weigh what they read, not what they put out: the other reading is far away, so the
    # comparison above would see a part that weighs the outputs
    n = min(T, 8)
    routed, _ = pt.moe(x[:n].double(), w64, "f.", {"router": {"top": K}, "shared": None}, forced=idx[:n])
    other = torch.zeros_like(routed)
    for tk in range(n):
        for j in range(K):
            e = int(idx[tk, j])
            other[tk] += scores[tk, e] * pt.gated_unit(x[tk:tk + 1].double(), w64[f"f.e{e}.gate"], w64[f"f.e{e}.up"],
                                                       w64[f"f.e{e}.down"])[0]
    assert float((routed - other).abs().max()) > 1e-2 * float(ref.abs().max())


def test_the_block_takes_the_pending_sum_and_hands_on_rounded_rows():
    """``output_norm_residual`` with a mixer that returns its input times two and a routed feed-forward: the
    residual after the block, and the rows it hands on, against the plain formulas."""
    from mini_infer_b200.config import part_class
    from mini_infer_b200.parts.base import BuiltLayer, Mixer, RoundedResidual
    W, T, E, K = 64, 19, 4, 2

    class Twice(Mixer):
        def forward(self, x, ctx, cache):
            return 2.0 * x.float()

    for dtype in ("float32", "bfloat16"):
        rt = runtime(dtype)
        g = torch.Generator().manual_seed(5)
        moe = part_class("feed_forward", "sparse_moe")({
            "hidden_size": W, "num_experts": E, "top_k": K, "expert_intermediate_size": 64, "shared_intermediate_size": 64,
            "scoring": "sigmoid", "weight_input": True, "router": "router", "expert": "e{e}.", "gate": "gate", "up": "up",
            "down": "down", "shared": "shared.", "shared_gate": "shared.sg"}, "f.")
        n1 = part_class("norm", "rmsnorm")({"size": W, "eps": 1e-5, "tensor": "n1"}, "")
        n2 = part_class("norm", "rmsnorm")({"size": W, "eps": 1e-5, "tensor": "n2"}, "")
        block = part_class("block", "output_norm_residual")({"residual_mult": 0.4}, "")
        t = {d.name: (torch.randn(*d.shape, generator=g) * (2.0 / d.shape[-1] ** 0.5)).to(torch.bfloat16)
             for d in moe.tensor_decls()}
        t["n1"], t["n2"] = (1 + 0.2 * torch.randn(W, generator=g)).to(torch.bfloat16), (1 + 0.2 * torch.randn(W, generator=g)).to(torch.bfloat16)
        for p in (moe, n1, n2, block):
            p.load(t, rt)
        moe.keep_routing = True
        layer = BuiltLayer("l", block, {"mixer": Twice({}, ""), "mixer_norm": n1, "feed_forward": moe, "feed_forward_norm": n2})
        hidden0 = torch.randn(T, W, generator=g)
        hidden = hidden0.to(DEV).clone()
        pending = block.forward(layer, hidden, None, None, {})
        rnd = pt.same if dtype == "float32" else pt.as_bfloat16
        w64 = {k: v.double() for k, v in t.items()}
        x = hidden0.double()
        x = x + 0.4 * pt.norm_plain(2.0 * rnd(x), w64["n1"], 1e-5)
        y, _ = pt.moe(rnd(x), w64, "f.", {"router": {"top": K}, "shared": {"ff": 64}}, rnd, forced=moe.last_routing[0].cpu())
        x = x + 0.4 * pt.norm_plain(y, w64["n2"], 1e-5)
        tol = 3e-5 if dtype == "float32" else 2e-2
        assert float((hidden.double().cpu() - x).abs().max()) <= tol * float(x.abs().max())
        if dtype == "float32":
            assert pending is None
        else:
            assert isinstance(pending, RoundedResidual) and torch.equal(pending.x, hidden.to(torch.bfloat16))
