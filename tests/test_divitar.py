"""Divitar through the engine against the plain implementation (GPU): every mechanism's kernels alone, whole prompts,
portions down to two tokens, token-by-token decoding through captured graphs, batches of unequal requests beside each
alone, pages and request slots used again, keys far away, at page borders and just inside and outside every block and
window (in prompts and in decoding), the first tokens, long decoding, odd sizes, and greedy generation through the
scheduler."""
import copy

import numpy as np
import pytest
import torch

import plain_divitar as pd
from divitar_helpers import (MIXED, ODD, ONE_LAYER, REAL, WIDE, as_numpy, assert_close, assert_same, make_engine, make_weights,
                             mixed_schedule, plain, plain_all, run_cut, tokens_of)

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(t, dtype):
    return t.to(device="cuda", dtype=DTYPES[dtype]).contiguous()


def rounded(t, dtype):
    return t.to(DTYPES[dtype]).double()


# ---- each mechanism's kernels alone ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rotation_of_neighbours_with_longer_cosines_and_keys_kept_as_they_came(dtype):
    """Pairs (2i, 2i + 1) and (i, i + dims/2), cosine and sine times a length, part of a head rotated; and the form
    that writes q and k rotated and the keys once more unrotated behind them."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    T = 37
    pos = torch.randint(0, 600, (T,), generator=g).int()       # angles are 32-bit: their rounding grows with the position
    tol = 2e-4 if dtype == "float32" else 3e-2
    for heads, width, dims, neighbours, length in ((3, 16, 16, True, 1.11), (2, 20, 6, True, 1.0), (1, 8, 8, True, 0.9),
                                                   (5, 12, 10, False, 1.25), (2, 6, 0, True, 1.3)):
        x = rounded(torch.randn(T, heads, width, generator=g), dtype)
        freqs = torch.tensor(pd.plain_frequencies(77.0, dims) if dims else [], dtype=torch.float32)
        f64 = freqs.double().numpy()
        if neighbours:
            ref = pd.rotate_neighbours(x.numpy(), pos.numpy(), f64, dims, length)
        else:       # the half layout has no length of its own in the plain code: lengthen the rotated part afterwards
            ref = pd.rotate_half(x.numpy(), pos.numpy(), f64, dims)
            ref[..., :dims] *= length
        src = dev(x.view(T, heads * width).float(), dtype)
        dst = torch.zeros(T, heads * width + 5, dtype=DTYPES[dtype], device="cuda")
        ops.rope_rows(src, 0, width, dst, 5, width, pos.cuda(), heads, width, dims, freqs.cuda(), neighbours=neighbours,
                      length=length)
        assert np.abs(dst[:, 5:].double().cpu().numpy() - ref.reshape(T, -1)).max() < tol, (heads, width, dims)
    H, G, D, dims = 4, 2, 12, 8
    x = rounded(torch.randn(T, H + G, D, generator=g), dtype)
    freqs = torch.tensor(pd.divided_frequencies(50.0, dims, 4.0), dtype=torch.float32)
    ref = pd.rotate_half(x.numpy(), pos.numpy(), freqs.double().numpy(), dims).reshape(T, -1)
    src = dev(torch.cat([x.view(T, -1).float(), torch.randn(T, 3, generator=g)], 1), dtype)      # gate columns behind q | k
    qkv = torch.full((T, (H + 2 * G) * D), float("nan"), dtype=DTYPES[dtype], device="cuda")
    ops.rope_rows(src, 0, D, qkv, 0, D, pos.cuda(), H + G, D, dims, freqs.cuda(), keep_col0=(H + G) * D, keep_head0=H)
    got = qkv.double().cpu().numpy()
    assert np.abs(got[:, :(H + G) * D] - ref).max() < tol
    assert np.array_equal(got[:, (H + G) * D:], x[:, H:].reshape(T, -1).numpy())       # the values: the keys, bit for bit


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_constant_on_what_a_norm_adds(dtype):
    """x += m * delta and x += m * norm(delta), with the row normalised for the next part or handed on as it is."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for width, pad in ((40, 3), (64, 4), (321, 3), (1000, 8), (4100, 4)):     # rows in registers, or staged
        x = torch.randn(9, width, generator=g) * 2
        y = rounded(torch.randn(9, width + pad, generator=g) * 5, dtype)[:, pad:]
        wp, wn = 1 + 0.3 * torch.randn(width, generator=g), 1 + 0.3 * torch.randn(width, generator=g)
        for post in (None, (wp.cuda(), 1e-3, 0.0)):
            for w in (None, wn.cuda()):
                xd = x.cuda()
                yd = dev(torch.cat([torch.zeros(9, pad), y.float()], 1), dtype)[:, pad:]
                out = torch.empty(9, width, dtype=DTYPES[dtype], device="cuda")
                ops.add_rmsnorm(xd, yd, None, post, w, 1e-4, 0.0, out, delta_scale=0.7)
                add = pd.rms_norm(y.numpy(), wp.numpy(), 1e-3) if post else y.numpy()
                x_ref = x.double().numpy() + 0.7 * add
                assert np.abs(xd.double().cpu().numpy() - x_ref).max() < 2e-6 * np.abs(x_ref).max()      # the stream stays 32-bit
                o_ref = pd.rms_norm(x_ref, wn.numpy(), 1e-4) if w is not None else x_ref
                tol = 1e-5 if dtype == "float32" else 1e-2
                assert np.abs(out.double().cpu().numpy() - o_ref).max() < tol * np.abs(o_ref).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_router_weights_over_their_sum_times_a_constant(dtype):
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    for rows, W, E, top, scale in ((19, 40, 7, 3, 2.5), (5, 64, 12, 1, 0.5), (33, 24, 4, 4, 1.0)):
        h = rounded(torch.randn(rows, W, generator=g), dtype)
        r = rounded(torch.randn(E, W, generator=g) * 0.5, dtype)
        ids, weights, gap = pd.route({"router": r.numpy()}, "", h.numpy(), top, scale)
        di = torch.empty(rows, top, dtype=torch.int32, device="cuda")
        dw = torch.empty(rows, top, dtype=torch.float32, device="cuda")
        ops.route_topk(dev(h.float(), dtype), dev(r.float(), dtype), top, "sigmoid", True, di, dw, 1e-20, scale)
        sure = gap > 1e-4
        assert sure.sum() > rows // 2
        order_got, order_ref = np.argsort(di.cpu().numpy(), 1), np.argsort(ids, 1)       # the chosen ones, in any order
        assert np.array_equal(np.take_along_axis(di.cpu().numpy(), order_got, 1)[sure], np.take_along_axis(ids, order_ref, 1)[sure])
        assert np.abs(np.take_along_axis(dw.cpu().numpy(), order_got, 1)[sure]
                      - np.take_along_axis(weights, order_ref, 1)[sure]).max() < 1e-5
        assert np.abs(dw.cpu().numpy().sum(1) - scale).max() < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_product_with_a_tokens_row_of_a_table(dtype):
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    for rows, n, vocab in ((21, 12, 50), (3, 7, 9), (300, 24, 40)):
        a = rounded(torch.randn(rows, n, generator=g) * 2, dtype)
        table = rounded(torch.randn(vocab, n, generator=g), dtype)
        tok = torch.randint(0, vocab, (rows,), generator=g).int()
        out = torch.empty(rows, n, dtype=DTYPES[dtype], device="cuda")
        ops.gate_mul(dev(a.float(), dtype), dev(table.float(), dtype), "gelu_tanh", out, b_rows=tok.cuda())
        ref = pd.gelu_tanh(a.numpy()) * table.numpy()[tok.numpy()]
        assert np.abs(out.double().cpu().numpy() - ref).max() < (1e-6 if dtype == "float32" else 5e-3) * np.abs(ref).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_relu_squared_in_the_products_epilogues(dtype):
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    for M, K, N in ((3, 64, 96), (40, 64, 96), (300, 128, 512), (17, 40, 24)):
        x = rounded(torch.randn(M, K, generator=g), dtype)
        w = rounded(torch.randn(N, K, generator=g) * K ** -0.5, dtype)
        got = ops.linear(dev(x.float(), dtype), dev(w.float(), dtype), None, "relu2").double().cpu().numpy()
        ref = np.maximum(x.numpy() @ w.numpy().T, 0.0) ** 2
        assert np.abs(got - ref).max() < (1e-5 if dtype == "float32" else 2e-2) * max(1.0, ref.max()), (M, K, N)


def _paged(k, v, ps, g):
    """Keys and values of one sequence scattered over pages in a random order; returns the pages and the block table."""
    T, G, D = k.shape
    pages = -(-T // ps)
    perm = torch.randperm(pages, generator=g)
    kp, vp = torch.zeros(pages, G, ps, D), torch.zeros(pages, G, ps, v.shape[2])
    for p in range(T):
        kp[perm[p // ps], :, p % ps] = k[p].float()
        vp[perm[p // ps], :, p % ps] = v[p].float()
    return kp, vp, perm.int().view(1, pages).cuda()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D, mask, sink", [(16, -50, False), (24, -37, False), (64, -150, False), (128, -64, False),
                                           (48, 45, True), (64, 100, True), (20, -1, False), (16, 1, True)])
def test_keys_at_the_edges_of_blocks_and_windows(D, mask, sink, dtype):
    """One sequence of 420 keys in pages of 8 or 16.  Every 29th key is made to stand out for every query, so a query's
    result hangs on exactly which of them it sees: as the queries walk on, such a key is the first one inside a block
    or window, the last one outside, at a page's border, the query's own, or hundreds of tokens back.  Every row of
    every kernel (general, general with the keys cut over blocks, tiled 32-bit, tiled tensor-core, TMA + tcgen05,
    decoding with and without splits) against the plain attention; ``mask`` < 0: blocks of -mask positions, > 0: a
    sliding window."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(8)
    T, H, G, scale = 420, 4, 2, 0.5
    ps = 16 if D >= 64 else 8          # the tensor-core forms of the decode kernel take pages of 16
    direction = torch.randn(D, generator=g)
    direction /= direction.norm()
    q = rounded(0.3 * torch.randn(T, H, D, generator=g) + 4.0 * direction, dtype)
    k = 0.3 * torch.randn(T, G, D, generator=g)
    k[::29] += 4.0 * direction
    k, v = rounded(k, dtype), rounded(torch.randn(T, G, D, generator=g), dtype)
    sinks = torch.tensor([0.5, -1.0, 2.0, 0.0]) if sink else None
    sees = (lambda i, j: pd.sees_block(i, j, -mask)) if mask < 0 else (lambda i, j: pd.sees_window(i, j, mask))
    ref = torch.from_numpy(pd.attention_rows(q.numpy(), k.numpy(), v.numpy(), scale, sees,
                                             None if sinks is None else sinks.numpy())).view(T, H * D)
    kp, vp, bt = _paged(k, v, ps, g)
    kd, vd = dev(kp, dtype), dev(vp, dtype)
    qd = dev(q.view(T, H * D).float(), dtype)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    sk = None if sinks is None else sinks.cuda()
    extra = {} if sinks is None else {"sinks": sk}
    tol = 1e-5 if dtype == "float32" else 2e-2

    def check(out, rows=slice(None), what=""):
        assert (out.double().cpu() - ref[rows]).abs().max() < tol, (what, D, mask)

    out = torch.zeros(T, H * D, dtype=DTYPES[dtype], device="cuda")
    ops.paged_attention_generic(qd, kd, vd, bt, seq, pos, out, H, G, D, ps, scale, mask, **extra)
    check(out, what="general")
    if D % 4 == 0:
        some = torch.zeros(120, H * D, dtype=DTYPES[dtype], device="cuda")
        part = torch.empty(120 * H * 4 * (D + 4), device="cuda")
        ops.paged_attention_generic(qd[300:], kd, vd, bt, seq[300:], pos[300:], some, H, G, D, ps, scale, mask, (4, 128), part, **extra)
        check(some, slice(300, 420), "general, keys cut")
    cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    start = torch.zeros(1, dtype=torch.int32, device="cuda")
    if dtype == "float32" and D % 16 == 0 and sinks is None:
        out2 = torch.zeros_like(out)
        ops.paged_prefill_f32(qd, kd, vd, bt, cu, start, out2, 0, 1, T, H, G, D, ps, scale, mask)
        check(out2, what="tiled 32-bit")
    if dtype == "bfloat16" and D % 8 == 0:
        if D % 16 == 0 or sinks is not None:      # without a sink or values of their own width the tiles are 16 wide
            out2 = torch.zeros_like(out)
            ops.paged_prefill_bf16(qd, kd, vd, bt, cu, start, out2, 0, 1, T, H, G, D, ps, scale, mask, **extra)
            check(out2, what="tiled tensor-core")
        if D in (64, 128) and sinks is None:
            out4 = torch.zeros_like(out)
            ops.paged_prefill_tc5(qd, kd, vd, bt, cu, start, out4, 0, 1, T, H, G, D, ps, scale, mask)
            ops.raise_if_kernel_errors()
            check(out4, what="TMA + tcgen05")
    # a portion of 120 rows behind 300 cached keys, the keys cut four ways over more blocks and merged
    cu2 = torch.tensor([300, T], dtype=torch.int32, device="cuda")
    start2 = torch.full((1,), 300, dtype=torch.int32, device="cuda")
    part = torch.empty(120 * H * 4 * (D + 4), device="cuda")
    if dtype == "float32" and D % 16 == 0 and sinks is None:
        out5 = torch.zeros_like(out)
        ops.paged_prefill_f32(qd, kd, vd, bt, cu2, start2, out5, 0, 1, 120, H, G, D, ps, scale, mask, (4, 128), part, pos, 300, 120)
        check(out5[300:], slice(300, T), "tiled 32-bit, keys cut")
    if dtype == "bfloat16" and D % 8 == 0 and (D % 16 == 0 or sinks is not None):
        out5 = torch.zeros_like(out)
        ops.paged_prefill_bf16(qd, kd, vd, bt, cu2, start2, out5, 0, 1, 120, H, G, D, ps, scale, mask, (4, 128), part, pos, 300, 120,
                               **extra)
        check(out5[300:], slice(300, T), "tiled tensor-core, keys cut")
    if dtype == "bfloat16" and D % 8 == 0:
        rows = list(range(0, T, 7)) + list(range(290, 320))     # decoding rows at many positions, as one batch
        n = len(rows)
        idx = torch.tensor(rows, device="cuda")
        for nsplit in (1, 4):
            out3 = torch.zeros(n, H * D, dtype=DTYPES[dtype], device="cuda")
            scratch = torch.empty(max(1, ops.decode_scratch_floats(n, H, D, nsplit)), device="cuda")
            counters = torch.zeros(n * H, dtype=torch.int32, device="cuda")
            ops.paged_decode_bf16(qd[idx].contiguous(), -1, -1, kd, vd, bt, seq[:n], pos[idx].contiguous(), pos[idx].contiguous(),
                                  out3, scratch, counters, H, G, D, ps, scale, mask, nsplit, **extra)
            check(out3, rows, f"decoding, {nsplit} splits")


# ---- whole models ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["attention", "latent", "dense", "routed", "side", "mixed", "odd"])
def test_whole_prompt_portions_and_single_tokens(name, dtype):
    """A whole prompt; portions of several sizes down to two tokens that end inside pages, blocks and windows; token
    by token from the first token on (decode steps, which replay captured graphs): all against the plain
    implementation.  One-layer models hold one mechanism each."""
    cfgd = {"mixed": MIXED, "odd": ODD}.get(name) or ONE_LAYER[name]
    w = make_weights(cfgd, 7)
    toks = tokens_of(cfgd, 75, 3)
    ref, _, close = plain_all(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype)
    whole = None
    for sizes in ([75], [13, 2, 9, 3, 16, 2, 30], [40] + [1] * 35, [2], [1]):
        got = run_cut(eng, toks, sizes)
        assert_close(got, ref, dtype, (name, sizes), close)
        if dtype == "bfloat16":
            whole = got if whole is None else whole
            assert_same(got, whole, (name, sizes))


def test_the_residual_stream_after_every_layer():
    """32-bit, a model cut after each of its layers: the last layer's stream shows in the logits of the shorter model
    (the final norm and the head are the same), so a fault is pinned to its layer."""
    w = make_weights(MIXED, 21)
    toks = tokens_of(MIXED, 40, 9)
    L = len(MIXED["layers"])
    for n in range(1, L + 1):
        cut = copy.deepcopy(MIXED)
        cut["layers"] = cut["layers"][:n]
        wn = {k: v for k, v in w.items() if not (k[0] == "l" and k[1].isdigit()) or int(k[1:k.index(".")]) < n}
        wn["side.embed"] = w["side.embed"][:, :n * MIXED["token_side"]["dim"]].contiguous()
        got = run_cut(make_engine(cut, wn, "float32"), toks, [17, 2, 21])
        assert (got - plain(cut, wn, toks)).abs().max() < 2e-4, n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_of_the_tiled_kernels(dtype):
    cfgd = WIDE
    w = make_weights(cfgd, 17, std=0.12)
    toks = tokens_of(cfgd, 200, 5)
    ref, _, close = plain_all(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype, page_size=16, num_pages=40, max_batched_tokens=256)
    for sizes in ([200], [100, 3, 64, 2, 31], [170] + [1] * 30):
        assert_close(run_cut(eng, toks, sizes), ref, dtype, sizes, close, tol32=1e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_as_wide_as_a_small_real_model(dtype):
    """Width 512, a prompt of 300 tokens: the products run on the TMA + tcgen05 kernels (relu squared in the epilogue,
    results added by the scaled norm), the experts in tiles over rows sorted by expert, attention of head size 64 on the
    tensor-core kernels for prompts and for decoding."""
    cfgd = REAL
    w = make_weights(cfgd, 19, std=0.1)
    toks = tokens_of(cfgd, 300, 5)
    ref, _, close = plain_all(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype, page_size=16, num_pages=40, max_batched_tokens=512)
    for sizes in ([300], [150, 2, 148], [270] + [1] * 30):
        assert_close(run_cut(eng, toks, sizes), ref, dtype, sizes, close, tol32=1e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype):
    """Six requests through three slots and a pool smaller than the requests together: portions of some beside single
    tokens of others; every logit equals the request's alone.  Freed pages are filled with NaN before they are used
    again."""
    cfgd = MIXED if name == "mixed" else ODD
    w = make_weights(cfgd, 9)
    lens = {"a": 70, "b": 33, "c": 58, "d": 2, "e": 47, "f": 64}
    seqs = {r: tokens_of(cfgd, n, 40 + i) for i, (r, n) in enumerate(lens.items())}
    plan = {"a": [30, 2, 1, 1, 1, 1, 1, 33], "b": [2, 20, 1, 1, 1, 8], "c": [50, 1, 1, 2, 1, 1, 1, 1], "d": [2],
            "e": [3, 1, 1, 1, 41], "f": [17, 40, 1, 1, 1, 1, 1, 1, 1]}
    assert all(sum(plan[r]) == lens[r] for r in lens)
    eng = make_engine(cfgd, w, dtype, num_pages=26, max_num_seqs=3, poison_freed_pages=True)
    got = mixed_schedule(eng, seqs, plan, list(lens))
    assert eng.pages_poisoned > 10
    for r in lens:
        ref, _, close = plain_all(cfgd, w, seqs[r])
        assert_close(got[r], ref, dtype, r, close)
        if dtype == "bfloat16":
            assert_same(got[r], run_cut(eng, seqs[r], [lens[r]]), r)


# ---- weights made so that a fault shows ------------------------------------------------------------------------
def _stand_out(cfgd):
    """Weights of a one-layer attention model in which token 5's key stands out for every query: a large entry in the
    token's row of the table, picked up by entry 0 of every key head, where every query has a constant (its bias)."""
    def tweak(t):
        D = cfgd["layers"][0]["mixer"]["dim"]
        t["embed"][5] *= 0.1
        t["embed"][5, 0] = 6.0
        t["l0.mix.q"] *= 0.2                      # the other scores stay small beside the marked one
        t["l0.mix.k"] *= 0.2
        t["l0.mix.k"][:, 0] = 0.0
        t["l0.mix.k"][0::D, 0] = 1.0
        t["l0.mix.q.b"][0::D] = 4.0
    return tweak


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_token_that_every_later_query_looks_for(dtype):
    """A one-layer attention model (no rotation of the entry that carries the mark) in which one token's key
    outweighs all others: it comes at positions that are first in a block, last in a block, and far back; rows after
    it change altogether when it drops out of sight at the block's end.  Whole, in portions and token by token."""
    from divitar_helpers import attn, config
    cfgd = config(64, 80, [attn(2, 1, 16, 40, 0.5, base=100.0, rot_dims=0, mlp=None)], side=None)
    w = make_weights(cfgd, 31, tweak=_stand_out(cfgd))
    toks = [t if t != 5 else 6 for t in tokens_of(cfgd, 170, 12)]
    for p in (39, 40, 81, 119, 120):
        toks[p] = 5
    ref = plain(cfgd, w, toks)
    # the mark matters: without the marked token in sight the row is another one
    other = plain(cfgd, w, [t if i != 81 else 7 for i, t in enumerate(toks)])
    assert (ref[100] - other[100]).abs().max() > 0.05 and (ref[125] - other[125]).abs().max() < 1e-9
    eng = make_engine(cfgd, w, dtype)
    for sizes in ([170], [39, 2, 40, 38, 2, 49], [118] + [1] * 52):
        assert_close(run_cut(eng, toks, sizes), ref, dtype, sizes)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_blocks_and_windows(dtype):
    """A short prompt and 200 tokens one by one: every block and window of the model passes over decoded tokens
    several times, and the cached rows of the first tokens drop out of the windows."""
    cfgd = MIXED
    w = make_weights(cfgd, 11)
    toks = tokens_of(cfgd, 220, 4)
    ref, _, close = plain_all(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype)
    assert_close(run_cut(eng, toks, [20] + [1] * 200), ref, dtype, "decode", close)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype):
    """Five prompts of unlike lengths through ``Engine.generate`` (three slots, prompts cut into portions of 16, a pool
    that holds less than all of them): the tokens are the plain implementation's greedy choices wherever its two best
    logits are further apart than rounding."""
    import cbis_b200 as cb
    from divitar_helpers import unrouted
    cfgd = MIXED if dtype == "float32" else unrouted(MIXED)      # bfloat16: rounding may flip an expert, so none there
    w = make_weights(cfgd, 13)
    prompts = [tokens_of(cfgd, n, 70 + n) for n in (3, 40, 1, 25, 33)]
    new = 12
    eng = make_engine(cfgd, w, dtype, num_pages=24, max_num_seqs=3, max_batched_tokens=64, prefill_chunk=16)
    outs = eng.generate(prompts, cb.SamplingParams(max_new_tokens=new))
    gap = 1e-3 if dtype == "float32" else 0.25
    checked = 0
    for p, o in zip(prompts, outs):
        assert len(o) == new
        seq = list(p)
        for tok in o:
            logits = plain(cfgd, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if top2[0] - top2[1] < gap:
                break                                   # a close call: from here on the sequences may part
            assert tok == int(logits.argmax()), (len(p), len(seq))
            seq.append(tok)
            checked += 1
    assert checked >= 5, checked          # some tokens were compared at all
    assert eng.scheduler.idle()
    again = eng.generate(prompts[:2], cb.SamplingParams(max_new_tokens=new))     # slots and pages used again
    assert again == outs[:2]
    warm = make_engine(cfgd, w, dtype, num_pages=24, max_num_seqs=3, max_batched_tokens=64, prefill_chunk=16)
    assert warm.warm_up() > 0
    assert warm.generate(prompts[:2], cb.SamplingParams(max_new_tokens=new)) == outs[:2]


# ---- trace replay through bin/trace_run -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_model_folder(dtype, tmp_path):
    """A Divitar folder (config.json, model.safetensors) through ``bin/trace_run``: a request whole; one with its last
    20 tokens one by one; one in portions down to two tokens; and four live requests in mixed steps through a pool
    smaller than the requests together, so that pages and request slots are used again."""
    import json
    import os

    from cbis_b200.weights.safetensors_io import write_safetensors
    from replay_helpers import Trace, read_logits, run_trace
    cfgd = MIXED
    w = make_weights(cfgd, 23)
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfgd, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: v.to(torch.bfloat16) for k, v in w.items()})
    lens = {"whole": 70, "tail": 50, "cut": 61, "m0": 40, "m1": 33, "m2": 64, "m3": 9, "m4": 21}
    seqs = {r: tokens_of(cfgd, n, 90 + i) for i, (r, n) in enumerate(lens.items())}
    t = Trace()
    t.step([("whole", seqs["whole"], range(70))], end=["whole"])
    t.step([("tail", seqs["tail"][:30], range(30))])
    for i in range(30, 50):
        t.step([("tail", seqs["tail"][i:i + 1], [0])], end=["tail"] if i == 49 else [])
    pos = 0
    for n in [16, 7, 2, 5, 2, 9, 3, 2, 15]:
        t.step([("cut", seqs["cut"][pos:pos + n], range(n))], end=["cut"] if pos + n == 61 else [])
        pos += n
    plan = {"m0": [30, 2, 1, 1, 6], "m1": [2, 20, 1, 10], "m2": [50, 1, 1, 12], "m3": [9], "m4": [3, 1, 17]}
    waiting, live, at, fed = list(plan), [], {}, {}
    while waiting or live:
        while waiting and len(live) < 4:
            r = waiting.pop(0)
            live.append(r); at[r] = 0; fed[r] = 0
        entries, ended = [], []
        for r in list(live):
            n = plan[r][at[r]]
            entries.append((r, seqs[r][fed[r]:fed[r] + n], range(n)))
            fed[r] += n; at[r] += 1
            if at[r] == len(plan[r]):
                ended.append(r); live.remove(r)
        t.step(entries, end=ended)
    bound = t.live_tokens_bound()
    assert bound < sum(-(-n // 64) * 64 for n in lens.values())
    out = str(tmp_path / "out")
    run_trace(t, folder, dtype, out, max_tokens=bound, page_size=8, env={"CBIS_POISON_FREED_PAGES": "1"})
    got = read_logits(t, out, cfgd["vocab"])
    for r, toks in seqs.items():
        rows = torch.from_numpy(np.stack([got[(r, p)][0] for p in range(len(toks))])).double()
        ref, _, close = plain_all(cfgd, w, toks)
        assert_close(rows, ref, dtype, r, close)
