"""Vatevik through the engine against the plain implementation (GPU): every mechanism's kernels alone, whole
prompts, portions down to two tokens, token-by-token decoding through captured graphs, batches of unequal requests
beside each alone, pages and request slots used again, page edges, far keys, the sink of score zero, blended values,
the first tokens, long decoding from a recurrent state, and greedy generation through the scheduler."""
import copy

import numpy as np
import pytest
import torch

import plain_vatevik as pv
from vatevik_helpers import (MIXED, ODD, WIDE, as_numpy, assert_close, assert_same, attn, config, dense, make_engine,
                             make_weights, mixed_schedule, plain, ret, run_cut, stretch, tokens_of, tolerance)

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(t, dtype):
    return t.to(device="cuda", dtype=DTYPES[dtype]).contiguous()


def rounded(t, dtype):
    return t.to(DTYPES[dtype]).double()


# ---- each mechanism's kernels alone ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_result_normalised_and_added_rows_handed_on_as_they_are(dtype):
    """x += norm(result); the next part gets x itself, rounded to its type (no norm before the part)."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for width, pad in ((40, 3), (40, 4), (321, 3), (1000, 8), (4100, 4)):     # rows in registers, or staged
        x = torch.randn(9, width, generator=g) * 2
        y = rounded(torch.randn(9, width + pad, generator=g) * 5, dtype)
        wb = 1 + 0.3 * torch.randn(width, generator=g)
        xd, yd = x.cuda(), dev(y.float(), dtype)[:, pad:]
        out = torch.empty(9, width, dtype=DTYPES[dtype], device="cuda")
        ops.add_rmsnorm(xd, yd, None, (wb.cuda(), 1e-3, 0.0), None, 0.0, 0.0, out)
        x_ref = x.double().numpy() + pv.rms_norm(y[:, pad:].numpy(), wb.numpy(), 1e-3)
        assert np.abs(xd.double().cpu().numpy() - x_ref).max() < 1e-5 * np.abs(x_ref).max()     # the stream stays 32-bit
        assert torch.equal(out, xd.to(DTYPES[dtype]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, D, V, dims", [(2, 16, 24, 16), (1, 12, 44, 6), (3, 48, 48, 0), (2, 100, 36, 50), (1, 300, 20, 300)])
def test_retention_recurrence_over_steps(H, D, V, dims, dtype):
    """Three requests of unlike lengths, one of them starting at a later position: whole, then each cut into steps
    of other sizes (also single rows) with the state carried in its slot; a decay of 1, a fast one and slow ones."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    lens, starts = [37, 5, 18], [0, 900, 3]
    T = sum(lens)
    qkv = rounded(torch.randn(T, 3 + 2 * H * D + H * V, generator=g), dtype)
    decays = [1.0, 0.5, 0.999755859375][:H] if H > 1 else [0.9873046875]
    freqs = pv.frequencies(31.0, dims) if dims else np.zeros(0)
    ks = D ** -0.5
    refs, at = [], 0
    for n, p0 in zip(lens, starts):
        r = slice(at, at + n)
        pos = np.arange(p0, p0 + n)
        q = qkv[r, 3:3 + H * D].view(n, H, D).numpy()
        k = qkv[r, 3 + H * D:3 + 2 * H * D].view(n, H, D).numpy()
        v = qkv[r, 3 + 2 * H * D:].view(n, H, V).numpy()
        if dims:
            q, k = pv.rotate(q, pos, freqs, dims), pv.rotate(k, pos, freqs, dims)
        refs.append(torch.from_numpy(pv.retention_rows(q, k * ks, v, decays)[0]).view(n, H * V))
        at += n
    ref = torch.cat(refs)
    fd = torch.tensor(freqs, dtype=torch.float64).float().cuda()
    om = torch.tensor([1.0 - d for d in decays], dtype=torch.float64).float().cuda()

    def run(cuts):
        """cuts: per step a list of (request, rows)."""
        state = torch.full((4, H * V * D + 5), float("nan"), device="cuda")
        state[:3].zero_()
        fed = [0, 0, 0]
        first = [0, lens[0], lens[0] + lens[1]]
        y_all = torch.zeros(T, H * V, dtype=torch.float64)
        for step in cuts:
            rows, cu, slots, pos = [], [0], [], []
            for r, n in step:
                rows += list(range(first[r] + fed[r], first[r] + fed[r] + n))
                pos += list(range(starts[r] + fed[r], starts[r] + fed[r] + n))
                fed[r] += n
                cu.append(cu[-1] + n)
                slots.append(r)
            idx = torch.tensor(rows)
            y = torch.empty(len(rows), H * V, dtype=torch.float32, device="cuda")
            ops.retention(dev(qkv[idx].float(), dtype), 3, 3 + H * D, 3 + 2 * H * D, torch.tensor(pos, dtype=torch.int32, device="cuda"),
                          fd, dims, ks, om, state, torch.tensor(slots, dtype=torch.int32, device="cuda"),
                          torch.tensor(cu, dtype=torch.int32, device="cuda"), len(slots), H, D, V, y,
                          max_seg_rows=max(n for _, n in step))        # steps of short segments take another form
            y_all[idx] = y.double().cpu()
        assert fed == lens
        return y_all

    tol = 2e-4 if dims else 2e-5        # an angle of 900 in 32-bit is good to 1e-4; the recurrence is 32-bit in both
    whole = run([[(0, 37), (1, 5), (2, 18)]])
    assert (whole - ref).abs().max() < tol * max(1.0, ref.abs().max().item())
    cut = run([[(0, 16), (2, 1)], [(2, 1), (1, 2), (0, 1)], [(0, 17), (2, 16)], [(1, 3)], [(0, 1)], [(0, 2)]])
    assert torch.equal(cut, whole)                  # rows walked in order from the state: the same bits however they are cut


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, D, V, dims, piece", [(3, 16, 24, 16, 32), (2, 48, 40, 24, 64), (1, 300, 20, 0, 32), (3, 64, 64, 64, 128)])
def test_long_segments_cut_into_pieces_that_run_side_by_side(H, D, V, dims, piece, dtype):
    """Segments longer than a piece, as long as one, a multiple of it, one row more and one row fewer, and a short
    one, from states that earlier rows left: the pieces' end states from zero, the start states one after the other
    and the second walk give what the walk in one piece gives, and leave the same state (a decay of 1 among them)."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(9)
    before = [5, 0, 40, 1, 0, 7]
    lens = [4 * piece + 9, piece, 3 * piece, 2 * piece + 1, 2 * piece - 1, 3]
    n_req = len(lens)
    decays = [1.0, 0.96875, 0.999755859375][:H] if H > 1 else [0.9873046875]
    freqs = pv.frequencies(10000.0, dims) if dims else np.zeros(0)
    ks = D ** -0.5
    fd = torch.tensor(freqs, dtype=torch.float64).float().cuda()
    om = torch.tensor([1.0 - d for d in decays], dtype=torch.float64).float().cuda()
    dp = ops.retention_piece_decays(decays).cuda()
    rows = [b + n for b, n in zip(before, lens)]
    qkv = [rounded(torch.randn(r, 2 * H * D + H * V, generator=g), dtype) for r in rows]
    refs, ends = [], []
    for x, r in zip(qkv, rows):
        pos = np.arange(r)
        q, k = x[:, :H * D].view(r, H, D).numpy(), x[:, H * D:2 * H * D].view(r, H, D).numpy()
        v = x[:, 2 * H * D:].view(r, H, V).numpy()
        if dims:
            q, k = pv.rotate(q, pos, freqs, dims), pv.rotate(k, pos, freqs, dims)
        o, S = pv.retention_rows(q, k * ks, v, decays)
        refs.append(torch.from_numpy(o).view(r, H * V))
        ends.append(S)

    def run(piece_rows):
        state = torch.zeros(n_req, H * V * D, device="cuda")
        out = []
        for part in (0, 1):                       # the rows before, then the long segments, all requests in one step
            segs = [(x[:b] if part == 0 else x[b:]) for x, b in zip(qkv, before)]
            live = [i for i, s in enumerate(segs) if s.shape[0]]
            cu = np.cumsum([0] + [segs[i].shape[0] for i in live])
            pos = np.concatenate([np.arange(segs[i].shape[0]) + (before[i] if part else 0) for i in live])
            y = torch.empty(int(cu[-1]), H * V, dtype=torch.float32, device="cuda")
            ops.retention(dev(torch.cat([segs[i] for i in live]).float(), dtype), 0, H * D, 2 * H * D,
                          torch.tensor(pos, dtype=torch.int32, device="cuda"), fd, dims, ks, om, state,
                          torch.tensor(live, dtype=torch.int32, device="cuda"), torch.tensor(cu, dtype=torch.int32, device="cuda"),
                          len(live), H, D, V, y, max_seg_rows=max(segs[i].shape[0] for i in live),
                          piece_decays=dp if part else None, piece_rows=piece_rows if part else 0)
            out.append((live, cu, y.double().cpu()))
        return out[1], state.double().cpu()

    (live, cu, y_cut), s_cut = run(piece)
    (_, _, y_one), s_one = run(0)
    tol = 2e-4 if dims else 2e-5
    for j, i in enumerate(live):
        ref = refs[i][before[i]:]
        scale = max(1.0, ref.abs().max().item())
        assert (y_one[cu[j]:cu[j + 1]] - ref).abs().max() < tol * scale
        assert (y_cut[cu[j]:cu[j + 1]] - ref).abs().max() < tol * scale
        assert (y_cut[cu[j]:cu[j + 1]] - y_one[cu[j]:cu[j + 1]]).abs().max() < 2e-5 * scale      # rounding only
        S = torch.from_numpy(np.ascontiguousarray(np.asarray(ends[i]).transpose(0, 2, 1))).reshape(-1)   # kept as [H][V][D]
        s_scale = max(1.0, S.abs().max().item())
        assert (s_cut[i] - S).abs().max() < tol * s_scale
        assert (s_cut[i] - s_one[i]).abs().max() < 2e-5 * s_scale
    short = live.index(5)                          # a segment inside one piece walks its rows once: the same bits
    assert torch.equal(y_cut[cu[short]:cu[short + 1]], y_one[cu[short]:cu[short + 1]])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_queries_and_keys_prepared_in_one_pass(dtype):
    """One norm over all of q and one over all of k, the rotation of every head, blended values: the one-pass kernel
    against the plain functions, and against the same steps as kernels of their own."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    for H, G, D, V, dims, norm, blend in ((3, 1, 10, 14, 6, True, 0.3), (4, 2, 16, 16, 16, True, None), (2, 2, 12, 8, 0, True, 0.8),
                                          (2, 1, 24, 8, 8, False, 0.5), (16, 4, 128, 64, 128, True, 0.25)):
        T, pad = 7, 5
        dq, dk, dv = H * D, G * D, G * V
        buf = rounded(torch.randn(T, pad + dq + dk + dv + 3, generator=g) * 3, dtype)
        other = rounded(torch.randn(T, dv + 2, generator=g), dtype)
        qw, kw = 1 + 0.3 * torch.randn(dq, generator=g), 1 + 0.3 * torch.randn(dk, generator=g)
        pos = torch.tensor([0, 1, 2, 40, 1000, 7, 333], dtype=torch.int32)
        freqs = pv.frequencies(77.0, dims, stretch(4.0, 1.0, 4.0, 64)) if dims else np.zeros(0)
        fd = torch.tensor(freqs, dtype=torch.float64).float().cuda()
        q, k = buf[:, pad:pad + dq].numpy(), buf[:, pad + dq:pad + dq + dk].numpy()
        v = buf[:, pad + dq + dk:pad + dq + dk + dv].numpy()
        if norm:
            q, k = pv.rms_norm(q, qw.numpy(), 1e-3), pv.rms_norm(k, kw.numpy(), 1e-3)
        q, k = q.reshape(T, H, D), k.reshape(T, G, D)
        if dims:
            q, k = pv.rotate(q, pos.numpy(), freqs, dims), pv.rotate(k, pos.numpy(), freqs, dims)
        if blend is not None:
            v = (1 - blend) * v + blend * other[:, 2:].numpy()
        ref = np.concatenate([q.reshape(T, dq), k.reshape(T, dk), v], axis=1)
        got = dev(buf.float(), dtype)
        od = dev(other.float(), dtype)[:, 2:]
        ops.qk_prepare(got, pad, H, pad + dq, G, D, qw.cuda() if norm else None, kw.cuda() if norm else None, 1e-3, pos.cuda(), fd,
                       dims, pad + dq + dk, dv, od if blend is not None else None, blend or 0.0)
        tol = 3e-4 if dtype == "float32" else 3e-2          # the angle 1000 in 32-bit is good to 1e-4
        assert np.abs(got[:, pad:pad + dq + dk + dv].double().cpu().numpy() - ref).max() < tol * max(1.0, np.abs(ref).max())
        assert torch.equal(got[:, :pad].double().cpu(), buf[:, :pad]) and torch.equal(got[:, -3:].double().cpu(), buf[:, -3:])
        # the same steps one kernel each
        two = dev(buf.float(), dtype)
        qv, kv, vv = two[:, pad:pad + dq], two[:, pad + dq:pad + dq + dk], two[:, pad + dq + dk:pad + dq + dk + dv]
        if norm:
            ops.rms_norm(qv, qw.cuda(), 1e-3, qv)
            ops.rms_norm(kv, kw.cuda(), 1e-3, kv)
        if dims:
            ops.rope_rows(two, pad, D, two, pad, D, pos.cuda(), H, D, dims, fd)
            ops.rope_rows(two, pad + dq, D, two, pad + dq, D, pos.cuda(), G, D, dims, fd)
        if blend is not None:
            ops.blend_rows(vv, od, blend, vv)
        assert (two.double() - got.double()).abs().max().item() < (1e-5 if dtype == "float32" else 3e-2) * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_kernels_with_a_sink_of_score_zero(dtype):
    """The general kernel, (bfloat16) the tiled one and the decode kernel over the same pages with 1 added to the
    softmax's denominator: grouped heads, values of another width than the keys, small scores (the 1 then holds most
    of the denominator at the first tokens), a request that starts at a later position beside one from position 0."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    ps, H, G = 8, 4, 2
    for D, V in ((16, 24), (40, 40), (48, 80), (128, 104), (12, 20)):
        lens = [70, 33]
        T = sum(lens)
        q = rounded(torch.randn(T, H * D, generator=g), dtype)
        k = rounded(torch.randn(T, G, D, generator=g), dtype)
        v = rounded(torch.randn(T, G, V, generator=g), dtype)
        scale = 0.3 / D ** 0.5
        n_pages = sum(-(-n // ps) for n in lens)
        perm = torch.randperm(n_pages, generator=g).tolist()
        kp, vp = torch.zeros(n_pages, G, ps, D), torch.zeros(n_pages, G, ps, V)
        bt = torch.full((2, 16), -1, dtype=torch.int32)
        refs, at, used = [], 0, 0
        for s, n in enumerate(lens):
            for p in range(n):
                if p % ps == 0:
                    bt[s, p // ps] = perm[used]
                    used += 1
                kp[bt[s, p // ps], :, p % ps] = k[at + p].float()
                vp[bt[s, p // ps], :, p % ps] = v[at + p].float()
            r = slice(at, at + n)
            refs.append(torch.from_numpy(pv.attention_rows(q[r].view(n, H, D).numpy(), k[r].numpy(), v[r].numpy(), scale)).view(n, H * V))
            at += n
        ref = torch.cat(refs)
        kd, vd = dev(kp, dtype), dev(vp, dtype)
        pos = torch.cat([torch.arange(n) for n in lens]).int().cuda()
        row_seq = torch.cat([torch.full((n,), s) for s, n in enumerate(lens)]).int().cuda()
        sk = torch.zeros(H, device="cuda")
        out = torch.zeros(T, H * V, dtype=DTYPES[dtype], device="cuda")
        ops.paged_attention_generic(dev(q.float(), dtype), kd, vd, bt.cuda(), row_seq, pos, out, H, G, D, ps, scale, 0,
                                    v_head_dim=V, sinks=sk)
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert (out.double().cpu() - ref).abs().max() < tol, (D, V)
        if dtype == "bfloat16" and D % 8 == 0 and V % 8 == 0:
            out2 = torch.zeros_like(out)
            cu = torch.tensor([0, lens[0], T], dtype=torch.int32, device="cuda")
            ops.paged_prefill_bf16(dev(q.float(), dtype), kd, vd, bt.cuda(), cu, torch.zeros(2, dtype=torch.int32, device="cuda"),
                                   out2, 0, 2, max(lens), H, G, D, ps, scale, 0, v_head_dim=V, sinks=sk)
            assert (out2.double().cpu() - ref).abs().max() < tol, (D, V, "tiled")
            last = torch.tensor([lens[0] - 1, T - 1, 0, lens[0]])           # each request's last row, and its first
            qd = dev(q[last].float(), dtype)
            rs = torch.tensor([0, 1, 0, 1], dtype=torch.int32, device="cuda")
            ps_ = torch.tensor([lens[0] - 1, lens[1] - 1, 0, 0], dtype=torch.int32, device="cuda")
            for nsplit in (1, 3):
                out3 = torch.zeros(4, H * V, dtype=DTYPES[dtype], device="cuda")
                scratch = torch.empty(max(1, ops.decode_scratch_floats(4, H, V, nsplit)), device="cuda")
                counters = torch.zeros(4 * H, dtype=torch.int32, device="cuda")
                ops.paged_decode_bf16(qd, -1, -1, kd, vd, bt.cuda(), rs, ps_, ps_, out3, scratch, counters, H, G, D, ps, scale,
                                      0, nsplit, v_head_dim=V, sinks=sk)
                assert (out3.double().cpu() - ref[last]).abs().max() < tol, (D, V, "decode", nsplit)


def test_decode_kernel_tensor_core_form_with_a_sink():
    """Head sizes 64 and 128 with values as wide as the keys on pages of 16 and 32 keys: the decode kernel's
    tensor-core form takes the 1 in the denominator, with the keys of a row in one part and split over several
    blocks; rows at the first positions (where the 1 holds most of the denominator), at a page's last key and its
    first, and far into the context."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(15)
    H, G = 4, 2
    for D, ps in ((64, 16), (128, 16), (64, 32)):
        n = 300
        q = rounded(torch.randn(n, H * D, generator=g), "bfloat16")
        k = rounded(torch.randn(n, G, D, generator=g), "bfloat16")
        v = rounded(torch.randn(n, G, D, generator=g), "bfloat16")
        scale = 0.3 / D ** 0.5
        pages = -(-n // ps)
        perm = torch.randperm(pages, generator=g)
        kp, vp = torch.zeros(pages, G, ps, D), torch.zeros(pages, G, ps, D)
        for p in range(n):
            kp[perm[p // ps], :, p % ps] = k[p].float()
            vp[perm[p // ps], :, p % ps] = v[p].float()
        ref = torch.from_numpy(pv.attention_rows(q.view(n, H, D).numpy(), k.numpy(), v.numpy(), scale)).view(n, H * D)
        rows = torch.tensor([0, 1, ps - 1, ps, 2 * ps, 127, 128, 255, 256, n - 1])
        qd = dev(q[rows].float(), "bfloat16")
        pos = rows.int().cuda()
        seq = torch.zeros(len(rows), dtype=torch.int32, device="cuda")
        bt = perm.int().view(1, pages).cuda()
        sk = torch.zeros(H, device="cuda")
        for nsplit in (1, 3):
            out = torch.zeros(len(rows), H * D, dtype=torch.bfloat16, device="cuda")
            scratch = torch.empty(max(1, ops.decode_scratch_floats(len(rows), H, D, nsplit)), device="cuda")
            counters = torch.zeros(len(rows) * H, dtype=torch.int32, device="cuda")
            ops.paged_decode_bf16(qd, -1, -1, dev(kp, "bfloat16"), dev(vp, "bfloat16"), bt, seq, pos, pos, out, scratch, counters,
                                  H, G, D, ps, scale, 0, nsplit, v_head_dim=D, sinks=sk)
            assert (out.double().cpu() - ref[rows]).abs().max() < 2e-2, (D, ps, nsplit)
            plain = torch.zeros_like(out)              # without the sink the first rows differ by far more
            ops.paged_decode_bf16(qd, -1, -1, dev(kp, "bfloat16"), dev(vp, "bfloat16"), bt, seq, pos, pos, plain, scratch, counters,
                                  H, G, D, ps, scale, 0, nsplit)
            assert (plain.double().cpu() - ref[rows])[:2].abs().max() > 0.2, (D, ps, nsplit)


# ---- each mechanism as a model of one layer, and the mixed models -------------------------------------------
ONE_LAYER = {
    "retention": config(48, 50, [ret(2, 16, 8, [0.95, 0.999], base=40.0, rot_dims=12, mlp=dense(32))]),
    "attention": config(48, 50, [attn(4, 2, 8, 16, 0.3, base=60.0, rot_dims=6, scaling=stretch(4.0, 1.0, 2.0, 16), mlp=dense(32))]),
    "blended": config(48, 50, [attn(2, 1, 8, 16, 0.3, v_mix=True, mlp=None), attn(3, 1, 16, 16, 0.2, rot_dims=8, v_mix=True, mlp=dense(24))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["retention", "attention", "blended", "mixed", "odd"])
def test_whole_prompt_portions_and_single_tokens(name, dtype):
    """A whole prompt; portions of several sizes down to two tokens that end inside pages; token by token (decode
    steps, which replay captured graphs): all against the plain implementation."""
    cfgd = {"mixed": MIXED, "odd": ODD}.get(name) or ONE_LAYER[name]
    w = make_weights(cfgd, 7)
    toks = tokens_of(cfgd, 75, 3)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype)
    whole = None
    for sizes in ([75], [13, 2, 9, 3, 16, 2, 30], [40] + [1] * 35, [1]):
        got = run_cut(eng, toks, sizes)
        assert_close(got, ref, dtype, (name, sizes))
        if dtype == "bfloat16":
            whole = got if whole is None else whole
            assert_same(got, whole, (name, sizes))


def test_the_residual_stream_after_every_layer():
    """32-bit, a model cut after each of its layers: the last layer's stream shows in the logits of the shorter model
    (the final norm and the head are the same), so a fault is pinned to its layer."""
    w = make_weights(MIXED, 21)
    toks = tokens_of(MIXED, 40, 9)
    for n in range(1, len(MIXED["layers"]) + 1):
        cut = copy.deepcopy(MIXED)
        cut["layers"] = cut["layers"][:n]
        if n == 5:                                   # the layer whose values the last one takes must still be there
            assert cut["layers"][2]["mixer"]["v_mix"]
        wn = {k: v for k, v in w.items() if not k.startswith("l") or int(k[1:k.index(".")]) < n}
        got = run_cut(make_engine(cut, wn, "float32"), toks, [17, 2, 21])
        assert (got - plain(cut, wn, toks)).abs().max() < 2e-4, n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_of_the_tiled_kernels(dtype):
    cfgd = WIDE
    w = make_weights(cfgd, 17, std=0.12)
    toks = tokens_of(cfgd, 200, 5)
    ref = plain(cfgd, w, toks)
    eng = make_engine(cfgd, w, dtype, page_size=16, num_pages=40, max_batched_tokens=256)
    for sizes in ([200], [100, 3, 64, 2, 31], [170] + [1] * 30):
        assert_close(run_cut(eng, toks, sizes), ref, dtype, sizes, tol32=1e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype):
    """Six requests through three slots and a pool smaller than the requests together: portions of some beside single
    tokens of others; every logit equals the request's alone.  Freed pages are filled with NaN before they are used
    again, and a slot's recurrent state starts from zero."""
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
        assert_close(got[r], plain(cfgd, w, seqs[r]), dtype, r)
        if dtype == "bfloat16":
            assert_same(got[r], run_cut(eng, seqs[r], [lens[r]]), r)


# ---- weights made so that a fault shows ------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_beside_the_sink(dtype):
    """700 keys in pages of 8 with 1 in the denominator: the keys at positions 3, 63 and 64 (inside the first page,
    and on both sides of a page's border) are made to stand out for every query, so that they hold most of the
    softmax's weight hundreds of tokens later; a kernel that loses a far key, or takes the page beside it, gives
    another result altogether."""
    from cbis_b200.kernels import ops
    g = torch.Generator().manual_seed(6)
    T, H, G, D, V, ps, scale = 700, 2, 1, 16, 24, 8, 0.5
    direction = torch.randn(D, generator=g)
    direction /= direction.norm()
    q = rounded(0.3 * torch.randn(T, H, D, generator=g) + 4.0 * direction, dtype)
    k = 0.3 * torch.randn(T, G, D, generator=g)
    for far in (3, 63, 64):
        k[far, 0] += 4.0 * direction
    k, v = rounded(k, dtype), rounded(torch.randn(T, G, V, generator=g), dtype)
    rows = list(range(600, 700))
    ref = torch.from_numpy(pv.attention_rows(q.numpy(), k.numpy(), v.numpy(), scale))[rows].view(len(rows), H * V)
    alone = pv.softmax_plus_one((k[:700, 0].numpy() @ q[699, 0].numpy()) * scale)
    assert alone[[3, 63, 64]].sum() > 0.8                     # the far keys hold the weight
    pages = -(-T // ps)
    perm = torch.randperm(pages, generator=g)
    kp, vp = torch.zeros(pages, G, ps, D), torch.zeros(pages, G, ps, V)
    for p in range(T):
        kp[perm[p // ps], :, p % ps] = k[p].float()
        vp[perm[p // ps], :, p % ps] = v[p].float()
    bt = perm.int().view(1, pages).cuda()
    qd = dev(q.view(T, H * D).float(), dtype)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    sk = torch.zeros(H, device="cuda")
    tol = 1e-5 if dtype == "float32" else 2e-2
    out = torch.zeros(T, H * V, dtype=DTYPES[dtype], device="cuda")
    ops.paged_attention_generic(qd, dev(kp, dtype), dev(vp, dtype), bt, seq, pos, out, H, G, D, ps, scale, 0, v_head_dim=V, sinks=sk)
    assert (out[rows].double().cpu() - ref).abs().max() < tol
    some = torch.zeros(100, H * V, dtype=DTYPES[dtype], device="cuda")
    part = torch.empty(100 * H * 4 * (V + 4), device="cuda")
    ops.paged_attention_generic(qd[600:], dev(kp, dtype), dev(vp, dtype), bt, seq[600:], pos[600:], some, H, G, D, ps, scale, 0,
                                (3, 256), part, v_head_dim=V, sinks=sk)
    assert (some.double().cpu() - ref).abs().max() < tol
    if dtype == "bfloat16":
        out2 = torch.zeros_like(out)
        cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
        ops.paged_prefill_bf16(qd, dev(kp, dtype), dev(vp, dtype), bt, cu, torch.zeros(1, dtype=torch.int32, device="cuda"), out2,
                               0, 1, T, H, G, D, ps, scale, 0, v_head_dim=V, sinks=sk)
        assert (out2[rows].double().cpu() - ref).abs().max() < tol
        for nsplit in (1, 4):
            out3 = torch.zeros(1, H * V, dtype=DTYPES[dtype], device="cuda")
            scratch = torch.empty(max(1, ops.decode_scratch_floats(1, H, V, nsplit)), device="cuda")
            counters = torch.zeros(H, dtype=torch.int32, device="cuda")
            ops.paged_decode_bf16(qd[699:], -1, -1, dev(kp, dtype), dev(vp, dtype), bt, seq[:1], pos[699:], pos[699:], out3, scratch,
                                  counters, H, G, D, ps, scale, 0, nsplit, v_head_dim=V, sinks=sk)
            assert (out3.double().cpu() - ref[-1:]).abs().max() < tol, nsplit


def test_the_sink_the_norms_over_whole_projections_and_the_blend_show():
    """Without the 1 in the denominator, with a norm per head instead of one over the whole projection, with the blend
    left out, or with the rotation's slow pairs not slowed down, the plain logits move by far more than the tolerance;
    the engine agrees with the right ones, in prompts over many pages and decoded one by one."""
    cfgd = config(24, 40, [attn(2, 1, 8, 12, 0.4, base=100.0, scaling=stretch(8.0, 1.0, 4.0, 32), v_mix=True, mlp=None),
                           attn(4, 1, 8, 12, 0.4, base=10.0, rot_dims=4, v_mix=True, mlp=None)])
    w = make_weights(cfgd, 8)
    toks = tokens_of(cfgd, 300, 4)
    ref = plain(cfgd, w, toks)
    wn = as_numpy(w)
    keep = (pv.softmax_plus_one, pv.rms_norm, pv.frequencies)
    try:
        pv.softmax_plus_one = lambda s: np.exp(s - s.max()) / np.exp(s - s.max()).sum()
        assert np.abs(pv.forward(cfgd, wn, toks[:20])[0] - ref[:20].numpy()).max() > 1e-2       # (among hundreds of keys it drowns)
        pv.softmax_plus_one = keep[0]
        def per_head(x, wt, eps):      # queries are 16 and 32 wide here, the stream 24
            if x.shape[-1] in (16, 32):
                return keep[1](x.reshape(len(x), -1, 8), 1.0, eps).reshape(x.shape) * wt
            return keep[1](x, wt, eps)
        pv.rms_norm = per_head
        assert np.abs(pv.forward(cfgd, wn, toks[:20])[0] - ref[:20].numpy()).max() > 1e-2
        pv.rms_norm = keep[1]
        pv.frequencies = lambda base, dims, scaling=None: keep[2](base, dims, None)
        assert np.abs(pv.forward(cfgd, wn, toks[:60])[0] - ref[:60].numpy()).max() > 1e-2
    finally:
        pv.softmax_plus_one, pv.rms_norm, pv.frequencies = keep
    unblended = copy.deepcopy(w)
    unblended["l1.mix.vmix"] = torch.zeros(())
    assert (plain(cfgd, unblended, toks[:20]) - ref[:20]).abs().max() > 1e-2
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(cfgd, w, dtype, num_pages=64, max_batched_tokens=512)
        for sizes in ([300], [97, 2, 64, 17], [250] + [1] * 50):
            assert_close(run_cut(eng, toks, sizes), ref, dtype, sizes)


def test_far_tokens_held_by_a_slow_decay_and_long_decoding():
    """Retention whose decays are near one: the logits 300 tokens later still depend on the first token, in a whole
    prompt, in portions, and when the last 150 tokens are decoded one by one; the rounded decay's lost digits do not
    add up."""
    cfgd = config(32, 40, [ret(2, 8, 12, [0.998291015625, 0.999755859375], base=1000.0, rot_dims=8, mlp=None)])
    w = make_weights(cfgd, 8)
    toks = tokens_of(cfgd, 300, 4)
    ref = plain(cfgd, w, toks)
    changed = plain(cfgd, w, [(toks[0] + 1) % 40] + toks[1:])
    assert (changed[-1] - ref[-1]).abs().max() > 1e-3
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(cfgd, w, dtype, num_pages=64, max_batched_tokens=512)
        for sizes in ([300], [97, 2, 64, 17], [150] + [1] * 150):
            got = run_cut(eng, toks, sizes)
            err = (got - ref).abs().max(1).values
            if dtype == "float32":
                assert err.max() < 2e-4, (sizes, err.max().item())
            else:
                tol = tolerance(dtype, ref)
                assert err.max() < tol and err.median() < tol / 4, (sizes, err.max().item(), err.median().item())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_cut_into_pieces_beside_decoding_rows(dtype):
    """One long segment beside five single rows from states of their own, the piece size chosen by the step: the long
    one is cut (the step counts as one long walk), the single rows walk as ever, and all agree with the uncut step."""
    from cbis_b200.kernels import ops
    H, D, V, n = 3, 32, 48, 300
    g = torch.Generator().manual_seed(12)
    decays = [1.0, 0.9375, 0.998291015625]
    lens = [1, 1, n, 1, 1, 1]
    T = sum(lens)
    assert ops.retention_piece_rows(n, len(lens), H, D, V, total_rows=T) > 0
    qkv = dev(torch.randn(T, 2 * H * D + H * V, generator=g), dtype)
    freqs = torch.tensor(pv.frequencies(10000.0, D), dtype=torch.float64).float().cuda()
    om = torch.tensor([1.0 - d for d in decays], dtype=torch.float64).float().cuda()
    dp = ops.retention_piece_decays(decays).cuda()
    cu = torch.tensor(np.cumsum([0] + lens), dtype=torch.int32, device="cuda")
    pos = torch.cat([torch.arange(m) + (0 if m > 1 else 77 + i) for i, m in enumerate(lens)]).to(torch.int32).cuda()
    slots = torch.tensor([4, 0, 2, 5, 1, 3], dtype=torch.int32, device="cuda")
    state0 = torch.randn(6, H * V * D, generator=g).cuda()
    state0[2].zero_()
    out = []
    for piece_rows in (None, 0):
        state = state0.clone()
        y = torch.empty(T, H * V, dtype=torch.float32, device="cuda")
        ops.retention(qkv, 0, H * D, 2 * H * D, pos, freqs, D, D ** -0.5, om, state, slots, cu, len(lens), H, D, V, y,
                      max_seg_rows=n, piece_decays=dp, piece_rows=piece_rows)
        out.append((y.double().cpu(), state.double().cpu()))
    (y_cut, s_cut), (y_one, s_one) = out
    assert (y_cut - y_one).abs().max() < 2e-5 * max(1.0, y_one.abs().max().item())
    assert (s_cut - s_one).abs().max() < 2e-5 * max(1.0, s_one.abs().max().item())
    single = [i for i in range(T) if not 2 <= i < 2 + n]
    assert torch.equal(y_cut[single], y_one[single])            # a single row is one piece: the same bits
    assert not torch.equal(s_one, state0.double().cpu())


def test_a_long_prompt_whose_retention_runs_in_pieces():
    """A prompt long enough that the engine cuts its retention segments into pieces: whole, in two long portions (the
    second from the state the first left), after a short portion, and in portions too short to be cut, all give the
    plain implementation's logits; one head never forgets, one forgets within a piece."""
    from cbis_b200.kernels import ops
    n = 5 * ops.RETENTION_PIECES_FROM + 37
    cfgd = config(48, 50, [ret(3, 16, 24, [1.0, 0.96875, 0.9990234375], base=1000.0, mlp=dense(32)),
                           attn(2, 1, 16, 16, 0.25, mlp=None),
                           ret(2, 24, 16, [0.999755859375, 0.9], rot_dims=8, mlp=dense(24))])
    w = make_weights(cfgd, 21)
    toks = tokens_of(cfgd, n, 6)
    ref = plain(cfgd, w, toks)
    half = 2 * ops.RETENTION_PIECES_FROM + 1
    for dtype in ("float32", "bfloat16"):
        eng = make_engine(cfgd, w, dtype, page_size=16, num_pages=-(-n // 16) + 4, max_batched_tokens=n + 8)
        for sizes in ([n], [half, n - half], [5, n - 5], [200], [100]):       # the last: portions too short to be cut
            got = run_cut(eng, toks, sizes)
            err = (got - ref).abs().max(1).values
            if dtype == "float32":
                assert err.max() < 3e-4, (sizes, err.max().item())
            else:
                tol = tolerance(dtype, ref)
                assert err.max() < tol and err.median() < tol / 4, (sizes, err.max().item(), err.median().item())


# ---- generation through the scheduler --------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype):
    """Five prompts of unlike lengths through ``Engine.generate`` (three slots, prompts cut into portions of 16, a pool
    that holds less than all of them): the tokens are the plain implementation's greedy choices wherever its two best
    logits are further apart than rounding."""
    import cbis_b200 as cb
    cfgd = MIXED
    w = make_weights(cfgd, 13)
    prompts = [tokens_of(cfgd, n, 70 + n) for n in (3, 40, 1, 25, 33)]
    new = 12
    eng = make_engine(cfgd, w, dtype, num_pages=24, max_num_seqs=3, max_batched_tokens=64, prefill_chunk=16)
    outs = eng.generate(prompts, cb.SamplingParams(max_new_tokens=new))
    gap = 1e-3 if dtype == "float32" else 0.25
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
    assert eng.scheduler.idle()
    again = eng.generate(prompts[:2], cb.SamplingParams(max_new_tokens=new))     # slots, pages and states used again
    assert again == outs[:2]
    warm = make_engine(cfgd, w, dtype, num_pages=24, max_num_seqs=3, max_batched_tokens=64, prefill_chunk=16)
    assert warm.warm_up() > 0
    assert warm.generate(prompts[:2], cb.SamplingParams(max_new_tokens=new)) == outs[:2]


# ---- trace replay through bin/trace_run -------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_of_a_model_folder(dtype, tmp_path):
    """A Vatevik folder (config.json, model.safetensors) through ``bin/trace_run``: a request whole; one with its last
    20 tokens one by one; one in portions down to two tokens; and four live requests in mixed steps through a pool
    smaller than the requests together, so that pages and state slots are used again."""
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
        assert_close(rows, plain(cfgd, w, toks), dtype, r)
